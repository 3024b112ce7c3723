"""Vufizen, Gositar or Banelix beside Qwen2, or Pibavik beside Banelix, at equal layer sizes: whole prompt steps and decode
steps, and the designs' own kernels one by one against their rooflines.

    python -m infero_b200.tools.design_bench [--design vufizen|gositar|banelix|pibavik] [--sizes s,m] [--prompt 2048] [--context 2048]
                                             [--batch 8] [--layers 8]

(also ``bench.py --designs``).  Random weights made on the device, bf16.  Per size two models of the same width
and depth: Vufizen (HGRN2 and differential-attention layers alternating, routed experts with a shared one) and
Qwen2 with the same head count, a head as wide as both maps together, and a feed-forward as wide as what one token
uses of the experts.  Steps are timed with CUDA events after warm-up, an L2 flush between timed steps; kernels are
timed alone the same way.  One JSON line at the end.

Gositar (``--design gositar``): latent attention in every layer (both mixer types alternating), dense squared-relu and
group-routed expert feed-forwards alternating, four residual streams; beside Qwen2 with the same head count, heads of
128, a quarter as many kv heads, and a feed-forward as wide as what one token uses on average.

Banelix (``--design banelix``): parallel layers (causal attention whose values are its keys beside a gated linear
recurrence) and windowed attention layers with a sink alternating, every second attention layer reading the keys and
values of the one before it; beside Qwen2 with the same width, head counts, heads of 128 and feed-forward.

Pibavik (``--design pibavik``): of every four layers one parallel layer (gated, normed window attention beside a state-space
recurrence), one window attention layer with a distance bias, one latent attention layer and one attention layer that reads
the keys and values of the one two before it, all with experts chosen by sigmoid scores and a shared expert; beside Banelix,
the closest of the other designs (parallel layers with a recurrence, window attention, borrowed caches), with the same width,
depth, head counts, window, recurrence width and a dense feed-forward as wide as what one token uses of the experts.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import types

SIZES = {
    "t": dict(width=256, heads=4, kv=2, dim=32, vdim=64, experts=4, top=2, ff=64, shared=128, vocab=1000),     # for tests
    "s": dict(width=1024, heads=8, kv=2, dim=64, vdim=128, experts=16, top=4, ff=512, shared=1024, vocab=32000),
    "m": dict(width=2048, heads=16, kv=4, dim=64, vdim=128, experts=32, top=4, ff=768, shared=1536, vocab=32000),
    "l": dict(width=4096, heads=32, kv=8, dim=64, vdim=128, experts=64, top=8, ff=768, shared=2048, vocab=32000),
}


GOSITAR_SIZES = {
    "t": dict(width=256, heads=4, dim=32, rot=16, vdim=32, rank=64, experts=4, top=2, groups=(2, 1), ff=64, shared=128, dense=512,
              streams=2, vocab=1000),                                                                         # for tests
    "s": dict(width=1024, heads=8, dim=64, rot=32, vdim=64, rank=256, experts=16, top=4, groups=(4, 2), ff=512, shared=1024,
              dense=4096, streams=4, vocab=32000),
    "m": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, rank=512, experts=32, top=4, groups=(4, 2), ff=768, shared=1536,
              dense=6144, streams=4, vocab=32000),
    "l": dict(width=4096, heads=32, dim=128, rot=64, vdim=128, rank=512, experts=64, top=8, groups=(8, 4), ff=768, shared=2048,
              dense=8192, streams=4, vocab=32000),
}


def gositar_config(z, layers):
    mix = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "kv_rank": z["rank"],
           "scale": (z["dim"] + z["rot"]) ** -0.5,
           "rot": {"base": 10000.0, "dims": z["rot"], "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    moe = {"kind": "moe", "expert": {"ff": z["ff"], "limit": 7.0}, "shared": {"ff": z["shared"], "limit": 7.0},
           "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}
    dense = {"kind": "dense", "ff": z["dense"]}
    return {"architecture": "Gositar", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "streams": z["streams"],
            "layers": [{"type": "latent_attention" if i % 2 == 0 else "latent_attention_2", "mixer": mix,
                        "mlp": dense if i % 2 == 0 else moe} for i in range(layers)]}


def qwen2_beside_gositar(z, layers):
    used = (z["dense"] * 2 // 3 + z["top"] * z["ff"] + z["shared"]) // 2          # (two matrices of `dense` against three)
    return {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": layers,
            "hidden_size": z["width"], "num_attention_heads": z["heads"], "num_key_value_heads": max(1, z["heads"] // 4),
            "head_dim": 128, "intermediate_size": -(-used // 64) * 64, "vocab_size": z["vocab"],
            "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False}


BANELIX_SIZES = {
    "t": dict(width=256, heads=4, kv=2, dim=64, window=48, rec=256, blocks=4, taps=4, ff=512, vocab=1000),            # for tests
    "s": dict(width=1024, heads=8, kv=2, dim=128, window=1024, rec=1024, blocks=8, taps=4, ff=4096, vocab=32000),
    "m": dict(width=2048, heads=16, kv=4, dim=128, window=1024, rec=2048, blocks=16, taps=4, ff=6144, vocab=32000),
    "l": dict(width=4096, heads=32, kv=8, dim=128, window=1024, rec=4096, blocks=32, taps=4, ff=11008, vocab=32000),
}


PIBAVIK_SIZES = {
    "t": dict(width=256, heads=4, kv=2, dim=64, window=48, ssd_heads=8, ssd_vdim=32, state=32, groups=2, taps=4, norm_groups=2,
              kv_rank=64, q_rank=96, experts=4, top=2, ff=128, shared=256, vocab=1000),                          # for tests
    "s": dict(width=1024, heads=8, kv=2, dim=128, window=1024, ssd_heads=16, ssd_vdim=64, state=64, groups=2, taps=4, norm_groups=2,
              kv_rank=256, q_rank=512, experts=16, top=2, ff=1024, shared=2048, vocab=32000),
    "m": dict(width=2048, heads=16, kv=4, dim=128, window=1024, ssd_heads=32, ssd_vdim=64, state=128, groups=4, taps=4, norm_groups=4,
              kv_rank=512, q_rank=768, experts=32, top=2, ff=1536, shared=3072, vocab=32000),
    "l": dict(width=4096, heads=32, kv=8, dim=128, window=1024, ssd_heads=64, ssd_vdim=64, state=128, groups=8, taps=4, norm_groups=8,
              kv_rank=512, q_rank=1536, experts=64, top=4, ff=2048, shared=2816, vocab=32000),
}


def pibavik_config(z, layers):
    D = z["dim"]
    left = {"heads": max(1, z["heads"] // 2), "kv_heads": max(1, z["kv"] // 2), "dim": D, "vdim": D, "scale": D ** -0.5,
            "mask": {"size": z["window"]}, "rot": {"base": 500000.0, "dims": D // 2}}
    right = {"heads": z["ssd_heads"], "vdim": z["ssd_vdim"], "state": z["state"], "groups": z["groups"], "conv": z["taps"],
             "norm_groups": z["norm_groups"]}
    par = {"left": left, "right": right, "left_scale": 0.7, "right_scale": 0.7}
    att = {"heads": z["heads"], "kv_heads": z["kv"], "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": z["window"]}}
    lat = {"heads": z["heads"], "dim": D, "vdim": D, "kv_rank": z["kv_rank"], "q_rank": z["q_rank"], "scale": D ** -0.5}
    mlp = {"kind": "moe", "expert": {"ff": z["ff"]}, "router": {"experts": z["experts"], "top": z["top"]}, "shared": {"ff": z["shared"]}}
    out = []
    for i in range(layers):
        if i % 4 == 0:
            out.append({"type": "parallel", "mixer": par, "mlp": mlp})
        elif i % 4 == 2:
            out.append({"type": "latent_attention", "mixer": lat, "mlp": mlp})
        else:
            out.append({"type": "attention", "mixer": dict(att, kv_from=i - 2) if i % 4 == 3 else att, "mlp": mlp})
    return {"architecture": "Pibavik", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": out}


def banelix_beside_pibavik(z, layers):
    b = dict(width=z["width"], heads=z["heads"], kv=z["kv"], dim=z["dim"], window=z["window"], rec=z["ssd_heads"] * z["ssd_vdim"],
             blocks=z["heads"], taps=z["taps"], ff=z["top"] * z["ff"] + z["shared"], vocab=z["vocab"])
    return banelix_config(b, layers)


def banelix_config(z, layers):
    D = z["dim"]
    left = {"heads": max(1, z["heads"] // 2), "kv_heads": max(1, z["kv"] // 2), "dim": D, "vdim": D, "scale": D ** -0.5,
            "rot": {"base": 500000.0, "dims": D // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    par = {"left": left, "right": {"width": z["rec"], "blocks": z["blocks"], "conv": z["taps"]}, "left_scale": 0.7, "right_scale": 0.7}
    att = {"heads": z["heads"], "kv_heads": z["kv"], "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": z["window"]},
           "rot": {"base": 10000.0, "dims": D, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    mlp = {"kind": "dense", "ff": z["ff"]}
    out = []
    for i in range(layers):
        if i % 2 == 0:
            out.append({"type": "parallel", "mixer": par, "mlp": mlp})
        else:
            out.append({"type": "attention", "mixer": dict(att, kv_from=i - 2) if i % 4 == 3 else att, "mlp": mlp})
    return {"architecture": "Banelix", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "residual_mult": 0.5, "layers": out}


def qwen2_beside_banelix(z, layers):
    return {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": layers,
            "hidden_size": z["width"], "num_attention_heads": z["heads"], "num_key_value_heads": z["kv"],
            "head_dim": z["dim"], "intermediate_size": z["ff"], "vocab_size": z["vocab"],
            "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False}


def vufizen_config(z, layers):
    mlp = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["ff"]},
           "shared": {"ff": z["shared"]}}
    att = {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["vdim"], "conv": 4, "diff": 0.5,
           "rot": {"base": 10000.0, "dims": z["dim"]}, "scale": z["dim"] ** -0.5}
    hg = {"heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"]}
    return {"architecture": "Vufizen", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5},
            "layers": [{"type": "hgrn2" if i % 2 == 0 else "attention", "mixer": hg if i % 2 == 0 else att, "mlp": mlp}
                       for i in range(layers)]}


def qwen2_config(z, layers):
    return {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": layers,
            "hidden_size": z["width"], "num_attention_heads": z["heads"], "num_key_value_heads": z["kv"],
            "head_dim": 2 * z["dim"], "intermediate_size": z["top"] * z["ff"] + z["shared"], "vocab_size": z["vocab"],
            "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False}


class _Timer:
    def __init__(self):
        import torch
        self.torch = torch
        self.flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn, reps=7, warmup=3, setup=None):
        torch = self.torch
        if setup is None:
            # a kernel alone: replayed from a captured graph, so that the host's share of a launch is not timed
            fn()
            torch.cuda.synchronize()
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    from infero_b200 import kernels as K
                    with K.stream_scope():
                        fn()
                fn = graph.replay
            except Exception:                          # noqa: BLE001  (something in fn cannot be captured: time it as it is)
                torch.cuda.synchronize()
        times = []
        for i in range(warmup + reps):
            if setup:
                setup()
            self.flush.fill_(i & 255)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= warmup:
                times.append(e0.elapsed_time(e1))
        times.sort()
        return times[len(times) // 2]


def time_model(cfg, prompt, context, batch, timer):
    import torch
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner, StepEntry
    from infero_b200.loading import random_model
    model, _ = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", generate_on_device=True)
    vocab = model.spec.vocab_size
    rng = random.Random(1)
    ps = 16
    toks = lambda n: [rng.randrange(vocab) for _ in range(n)]                   # noqa: E731
    runner = ModelRunner(model, EngineConfig(dtype="bfloat16", page_size=ps, num_pages=2 * (-(-prompt // ps)), max_seqs=2,
                                             ctx=prompt, max_batch_tokens=prompt, cuda_graphs=False))
    p = toks(prompt)

    def prefill():
        runner.step([StepEntry("p", p, [prompt - 1])])
    pre_ms = timer(prefill, setup=lambda: (("p" in runner.manager.requests) and runner.close("p"), runner.open("p")))
    del runner
    torch.cuda.empty_cache()
    steps = 24
    runner = ModelRunner(model, EngineConfig(dtype="bfloat16", page_size=ps, num_pages=batch * (-(-(context + 64) // ps)),
                                             max_seqs=batch, ctx=context + 64, max_batch_tokens=max(2048, batch),
                                             max_logit_rows=max(8, batch), cuda_graphs=True))
    rids = [f"d{i}" for i in range(batch)]
    for r in rids:
        runner.open(r)
        done = 0
        while done < context - steps:
            n = min(2048, context - steps - done)
            runner.step([StepEntry(r, toks(n), [])])
            done += n
    for _ in range(4):                                     # eager, captured, replayed
        runner.step([StepEntry(r, toks(1), [0]) for r in rids])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps - 4):
        runner.step([StepEntry(r, toks(1), [0]) for r in rids])
    e1.record()
    torch.cuda.synchronize()
    dec_ms = e0.elapsed_time(e1) / (steps - 4)
    out = {"prefill_tok_s": round(prompt / pre_ms * 1e3, 1), "prefill_ms": round(pre_ms, 3),
           "decode_tok_s": round(batch / dec_ms * 1e3, 1), "decode_ms_per_step": round(dec_ms, 4),
           "weight_mib": model.weight_bytes() >> 20, "graph_replays": runner.graph_replays}
    del runner, model
    torch.cuda.empty_cache()
    return out


def time_kernels(z, T, context, batch, timer, peaks):
    """The new design's kernels alone, each beside the kernel of the built-in decoder that does the like job."""
    import numpy as np
    import torch
    from infero_b200 import kernels as K
    from infero_b200.kernels import attention as A, diff_attention as DA, layer_ops as L, moe as M, tc_gemm
    from infero_b200.parts.linear import Linear
    dev, bf = "cuda:0", torch.bfloat16
    d, H, G, D, V = z["width"], z["heads"], z["kv"], z["dim"], z["vdim"]
    E, top, ff = z["experts"], z["top"], z["ff"]
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, dtype=bf, k=1.0: (torch.randn(s, generator=g, device=dev) * k).to(dtype)     # noqa: E731
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=dev)                 # noqa: E731
    hbm, tfl = peaks["hbm_gbs"], peaks["bf16_tflops"]
    rows = {}

    def note(name, ms, bytes_=0.0, flops=0.0):
        r = {"us": round(ms * 1e3, 1)}
        if bytes_:
            r["gb_s"] = round(bytes_ / ms / 1e6, 1)
            r["hbm_frac"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["tensor_frac"] = round(flops / ms / 1e9 / tfl, 3)
        rows[name] = r

    def batch_ctx(q_lens, pos0, ps=16):
        E_ = len(q_lens)
        per = [-(-(p + n) // ps) for p, n in zip(pos0, q_lens)]
        table = torch.full((E_, max(per)), -1, dtype=torch.int32)
        at = 0
        for e, n in enumerate(per):
            table[e, :n] = torch.arange(at, at + n, dtype=torch.int32)
            at += n
        qs = np.concatenate([[0], np.cumsum(q_lens)[:-1]])
        ctx = types.SimpleNamespace(
            n_entries=E_, n_tokens=int(sum(q_lens)), h_q_len=np.asarray(q_lens, dtype=np.int32), h_pos0=np.asarray(pos0, dtype=np.int32),
            tok_entry=i32(np.repeat(np.arange(E_), q_lens)), positions=i32(np.concatenate([p + np.arange(n) for p, n in zip(pos0, q_lens)])),
            entry_q_start=i32(qs), entry_q_len=i32(q_lens), entry_pos0=i32(pos0), entry_slot=i32(np.arange(E_)), kv_bound=None)
        return ctx, table.to(dev), at

    # ---- attention: prompt of T tokens, then `batch` single tokens at `context` -----------------------------------
    for label, q_lens, pos0 in (("prefill", [T], [0]), ("decode", [1] * batch, [context - 1] * batch)):
        ctx, table, pages = batch_ctx(q_lens, pos0)
        n = ctx.n_tokens
        kd, vd = rnd(pages, G, 16, 2 * D), rnd(pages, G, 16, V)
        kv = types.SimpleNamespace(k=kd, v=vd, page_size=16)
        padded = DA.as_plain_heads(bf, D, V, 16)
        q, out = rnd(n, 2 * H * D * (2 if padded else 1)), torch.empty(n, H * V, dtype=bf, device=dev)
        keys = sum(p + (n_ + 1) / 2 * 1 for p, n_ in zip(pos0, q_lens)) if label == "decode" else T / 2
        fl = 2.0 * H * (2 * D + 2 * V) * (T * T / 2 if label == "prefill" else batch * context)
        by = 2.0 * G * (2 * D + V) * (T if label == "prefill" else batch * context) + 2.0 * n * (2 * H * D + H * V)
        ms = timer(lambda: DA.paged_diff_attention(ctx, q, out, kv, table, H, G, D, V, None, D ** -0.5, 0.4, 1e-5, 0.5, q_padded=padded))
        note(f"diff_attention_{label}", ms, by, fl)
        # the built-in attention with a head as wide as both maps (2 D) and values of the same width
        Dq = 2 * D
        k2, v2 = rnd(pages, G, 16, Dq), rnd(pages, G, 16, Dq)
        q2, out2 = rnd(n, H * Dq), torch.empty(n, H * Dq, dtype=bf, device=dev)
        fl2 = 2.0 * H * 2 * Dq * (T * T / 2 if label == "prefill" else batch * context)
        by2 = 2.0 * G * 2 * Dq * (T if label == "prefill" else batch * context) + 4.0 * n * H * Dq
        ms = timer(lambda: A.attention_any(q2, out2, k2, v2, table, ctx.tok_entry, ctx.positions, H, G, Dq, 16, None, Dq ** -0.5,
                                           ctx.h_q_len, ctx.h_pos0, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_pos0))
        note(f"gqa_attention_{label}", ms, by2, fl2)
        if label == "prefill":      # the built-in kernel on the warp-level tensor cores (what head sizes other than 64 and 128 get)
            ms = timer(lambda: A.prefill(q2, out2, k2, v2, table, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_pos0, 1, 0,
                                         -(-T // 64), H, G, Dq, 16, None, Dq ** -0.5))
            note("gqa_attention_prefill_mma_sync", ms, by2, fl2)

    # ---- the recurrence ------------------------------------------------------------------------------------------
    for label, q_lens in (("prefill", [T]), ("decode", [1] * batch)):
        ctx, _, _ = batch_ctx(q_lens, [0] * len(q_lens))
        n = ctx.n_tokens
        proj = rnd(n, 2 * H * D + H * V, dtype=torch.float32)
        state = torch.zeros(len(q_lens), H, D, V, device=dev)
        fb, lo, wn = rnd(H * D, dtype=torch.float32), torch.rand(H * D, device=dev), torch.ones(V, device=dev)
        out = torch.empty(n, H * V, dtype=bf, device=dev)
        ms = timer(lambda: L.hgrn2_scan(proj, 0, H * D, 2 * H * D, fb, lo, wn, 1e-5, state, ctx.entry_q_start, ctx.entry_q_len,
                                        ctx.entry_slot, out, len(q_lens), H, D, V, q_lens=q_lens))
        note(f"hgrn2_scan_{label}", ms, 4.0 * n * (2 * H * D + H * V) + 2.0 * n * H * V + 8.0 * len(q_lens) * H * D * V)

    # ---- feed-forward: routed experts beside a dense SwiGLU of the width one token uses -----------------------------
    gu, dn = rnd(E, 2 * ff, d, k=0.05), rnd(E, d, ff, k=0.05)
    router = rnd(E, d, k=0.1)
    dense_ff = top * ff
    wgu, wdn = rnd(2 * dense_ff, d, k=0.05), rnd(d, dense_ff, k=0.05)
    for label, n in (("prefill", T), ("decode", batch)):
        h = rnd(n, d)
        y = torch.empty(n, d, device=dev)
        route = Linear(router)
        idx, w, _ = L.moe_select(route.forward(h, out_dtype=torch.float32), E, top)
        ms = timer(lambda: L.moe_select(route.forward(h, out_dtype=torch.float32), E, top))
        note(f"moe_route_{label}", ms, 2.0 * (n * d + E * d))
        used = min(E, n * top)
        ms = timer(lambda: M.experts(h, gu, dn, idx, w, None, None, y))
        note(f"moe_experts_{label}", ms, 2.0 * used * 3 * ff * d + 2.0 * n * d + 4.0 * n * d, 6.0 * n * top * ff * d)
        act = torch.empty(n, dense_ff, dtype=bf, device=dev)
        o = torch.empty(n, d, dtype=torch.float32, device=dev)

        def dense():
            if not tc_gemm.gemm_swiglu(h, wgu, act):
                K.swiglu(K.Partials(tc_gemm.partials(h, wgu)), act)
            tc_gemm.gemm(act, wdn, None, o)
        ms = timer(dense)
        note(f"dense_swiglu_{label}", ms, 2.0 * 3 * dense_ff * d + 6.0 * n * d, 6.0 * n * dense_ff * d)

    # ---- the small kernels -----------------------------------------------------------------------------------------
    x, yv, gl = rnd(T, d, dtype=torch.float32), rnd(T, d, dtype=torch.float32), rnd(T, d, dtype=torch.float32)
    gb, nw, hb = rnd(d, dtype=torch.float32), torch.ones(1, device=dev), torch.empty(T, d, dtype=bf, device=dev)
    ms = timer(lambda: L.gated_scalar_norm_add(x, yv, gl, gb, nw, 1e-5, hb))
    note("gated_norm_add_prefill", ms, T * d * (4 + 4 + 4 + 4 + 2))
    wv = torch.ones(d, device=dev)
    ms = timer(lambda: K.add_rmsnorm(x, yv, wv, 1e-5, hb))
    note("add_rmsnorm_prefill", ms, T * d * (4 + 4 + 4 + 2))
    ctx, table, pages = batch_ctx([T], [0])
    C = 2 * H * D + 2 * G * D + G * V
    proj, cw = rnd(T, C, dtype=torch.float32), rnd(4, C, dtype=torch.float32)
    st = torch.zeros(1, 3, C, device=dev)
    kd, vd = torch.empty(pages, G, 16, 2 * D, dtype=bf, device=dev), torch.empty(pages, G, 16, V, dtype=bf, device=dev)
    qn, inv = torch.ones(D, device=dev), torch.rand(D // 2, device=dev)
    qo = torch.empty(T, 2 * H * D, dtype=bf, device=dev)
    ms = timer(lambda: L.qkv_prepare(proj, cw, 4, st, qn, qn, 1e-5, inv, ctx.positions, ctx.tok_entry, ctx.entry_q_start,
                                     ctx.entry_slot, table, qo, kd, vd, 16, 2 * H, 2 * G, G, D, V))
    note("qkv_prepare_prefill", ms, T * C * (4 + 2))
    Dq = 2 * D
    qkv = rnd(T, (H + 2 * G) * Dq)
    k2, v2 = torch.empty(pages, G, 16, Dq, dtype=bf, device=dev), torch.empty(pages, G, 16, Dq, dtype=bf, device=dev)
    inv2 = torch.rand(Dq // 2, device=dev)
    ms = timer(lambda: K.rope_cache(qkv, ctx.positions, ctx.tok_entry, table, inv2, k2, v2, H, G, Dq, 16))
    note("rope_cache_prefill", ms, T * (H + 2 * G) * Dq * 2 * 2)
    return rows


def time_gositar_kernels(z, T, context, batch, timer, peaks):
    """Gositar's kernels alone, each beside the kernel of the built-in decoder that does the like job."""
    import numpy as np
    import torch
    from infero_b200 import kernels as K
    from infero_b200.kernels import attention as A, latent_attention as LA, layer_ops as L, moe as M, tc_gemm
    from infero_b200.parts.linear import Linear
    dev, bf = "cuda:0", torch.bfloat16
    d, H, D, R, V, C, S = z["width"], z["heads"], z["dim"], z["rot"], z["vdim"], z["rank"], z["streams"]
    E, top, ff = z["experts"], z["top"], z["ff"]
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, dtype=bf, k=1.0: (torch.randn(s, generator=g, device=dev) * k).to(dtype)     # noqa: E731
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=dev)                 # noqa: E731
    hbm, tfl = peaks["hbm_gbs"], peaks["bf16_tflops"]
    rows = {}

    def note(name, ms, bytes_=0.0, flops=0.0):
        r = {"us": round(ms * 1e3, 1)}
        if bytes_:
            r["gb_s"] = round(bytes_ / ms / 1e6, 1)
            r["hbm_frac"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["tensor_frac"] = round(flops / ms / 1e9 / tfl, 3)
        rows[name] = r

    def batch_ctx(q_lens, pos0, ps=16):
        E_ = len(q_lens)
        per = [-(-(p + n) // ps) for p, n in zip(pos0, q_lens)]
        table = torch.full((E_, max(per)), -1, dtype=torch.int32)
        at = 0
        for e, n in enumerate(per):
            table[e, :n] = torch.arange(at, at + n, dtype=torch.int32)
            at += n
        qs = np.concatenate([[0], np.cumsum(q_lens)[:-1]])
        ctx = types.SimpleNamespace(
            n_entries=E_, n_tokens=int(sum(q_lens)), h_q_len=np.asarray(q_lens, dtype=np.int32), h_pos0=np.asarray(pos0, dtype=np.int32),
            tok_entry=i32(np.repeat(np.arange(E_), q_lens)), positions=i32(np.concatenate([p + np.arange(n) for p, n in zip(pos0, q_lens)])),
            entry_q_start=i32(qs), entry_q_len=i32(q_lens), entry_pos0=i32(pos0), entry_slot=i32(np.arange(E_)), kv_bound=None)
        return ctx, table.to(dev), at

    G, Dq = max(1, H // 4), 128
    for label, q_lens, pos0 in (("prefill", [T], [0]), ("decode", [1] * batch, [context - 1] * batch)):
        ctx, table, pages = batch_ctx(q_lens, pos0)
        n = ctx.n_tokens
        pairs = T * T / 2 if label == "prefill" else batch * context           # (query, key) pairs per head
        keys = T if label == "prefill" else batch * context
        # ---- attention over the latent rows ------------------------------------------------------------------------
        kv = types.SimpleNamespace(k=rnd(pages, 1, 16, C + R), v=None, page_size=16, group=0)
        rows_h = -(-n // 128) * 128
        q_lat, q_rot = rnd(H, rows_h, C, dtype=torch.float32), rnd(H, rows_h, R, dtype=torch.float32)
        o_lat = torch.empty(H, rows_h, C, dtype=bf, device=dev)
        ms = timer(lambda: LA.attention(ctx, q_lat, q_rot, o_lat, kv, table, n, H, C, R, (D + R) ** -0.5))
        note(f"latent_attention_{label}", ms, 2.0 * (C + R) * keys + n * H * (4.0 * (C + R) + 2.0 * C), 2.0 * H * (2 * C + R) * pairs)
        rows[f"latent_attention_{label}"]["unabsorbed_tflops"] = round(2.0 * H * (D + R + V) * pairs / ms / 1e9, 1)
        # ---- the per-head products around it -----------------------------------------------------------------------
        q_plain, up_k = rnd(H, rows_h, D), rnd(H, C, D, k=0.05)
        ms = timer(lambda: LA.per_head_product(q_plain, up_k, q_lat, n))
        note(f"per_head_up_k_{label}", ms, 2.0 * H * C * D + H * rows_h * (2.0 * D + 4.0 * C), 2.0 * H * rows_h * C * D)
        up_v, val = rnd(H, V, C, k=0.05), torch.empty(H, rows_h, V, dtype=torch.float32, device=dev)
        ms = timer(lambda: LA.per_head_product(o_lat, up_v, val, n))
        note(f"per_head_up_v_{label}", ms, 2.0 * H * C * V + H * rows_h * (2.0 * C + 4.0 * V), 2.0 * H * rows_h * C * V)
        # ---- prepare beside rotary + cache append --------------------------------------------------------------------
        width = H * (D + R) + C + R + H
        proj, nw, fr = rnd(n, width, dtype=torch.float32), torch.ones(C, device=dev), torch.rand(R // 2, device=dev, dtype=torch.float64)
        ms = timer(lambda: LA.prepare(proj, 0, H * (D + R), nw, 1e-5, fr, "adjacent", 1.2, ctx.positions, ctx.tok_entry, table, kv.k,
                                      16, q_plain, q_rot, n, H, D, R, C))
        note(f"latent_prepare_{label}", ms, n * (4.0 * width + 2.0 * (C + R) + H * (2.0 * D + 4.0 * R)))
        gate, attn = proj[:, width - H:], torch.empty(n, H * V, dtype=bf, device=dev)
        ms = timer(lambda: LA.finish(val, gate, attn, n, H, V))
        note(f"latent_finish_{label}", ms, n * H * V * 6.0)
        # ---- the built-in attention: heads of 128, a quarter as many kv heads ----------------------------------------
        k2, v2 = rnd(pages, G, 16, Dq), rnd(pages, G, 16, Dq)
        q2, out2 = rnd(n, H * Dq), torch.empty(n, H * Dq, dtype=bf, device=dev)
        ms = timer(lambda: A.attention_any(q2, out2, k2, v2, table, ctx.tok_entry, ctx.positions, H, G, Dq, 16, None, Dq ** -0.5,
                                           ctx.h_q_len, ctx.h_pos0, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_pos0))
        note(f"gqa_attention_{label}", ms, 2.0 * G * 2 * Dq * keys + 4.0 * n * H * Dq, 2.0 * H * 2 * Dq * pairs)
        if label == "prefill":
            ms = timer(lambda: A.prefill(q2, out2, k2, v2, table, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_pos0, 1, 0,
                                         -(-T // 64), H, G, Dq, 16, None, Dq ** -0.5))
            note("gqa_attention_prefill_mma_sync", ms, 2.0 * G * 2 * Dq * keys + 4.0 * n * H * Dq, 2.0 * H * 2 * Dq * pairs)
        qkv = rnd(n, (H + 2 * G) * Dq)
        inv2 = torch.rand(Dq // 2, device=dev)
        ms = timer(lambda: K.rope_cache(qkv, ctx.positions, ctx.tok_entry, table, inv2, k2, v2, H, G, Dq, 16))
        note(f"rope_cache_{label}", ms, n * (H + 2 * G) * Dq * 2 * 2)

    # ---- feed-forward: group-routed experts with the clamped activation beside a dense SwiGLU of the width one token uses ----
    gu, dn = rnd(E, 2 * ff, d, k=0.05), rnd(E, d, ff, k=0.05)
    router, corr = rnd(E, d, k=0.1), rnd(E, dtype=torch.float32, k=0.1)
    dense_ff = top * ff
    wgu, wdn = rnd(2 * dense_ff, d, k=0.05), rnd(d, dense_ff, k=0.05)
    wup, wdown = rnd(z["dense"], d, k=0.05), rnd(d, z["dense"], k=0.05)
    act3 = ("glu_clamped", 7.0, 1.702)
    for label, n in (("prefill", T), ("decode", batch)):
        h = rnd(n, d)
        y = torch.empty(n, d, device=dev)
        route = Linear(router)
        idx, w = L.moe_select_grouped(route.forward(h, out_dtype=torch.float32), corr, E, top, *z["groups"])
        ms = timer(lambda: L.moe_select_grouped(route.forward(h, out_dtype=torch.float32), corr, E, top, *z["groups"]))
        note(f"moe_route_grouped_{label}", ms, 2.0 * (n * d + E * d))
        used = min(E, n * top)
        ms = timer(lambda: M.experts(h, gu, dn, idx, w, None, None, y, act3))
        note(f"moe_experts_clamped_{label}", ms, 2.0 * used * 3 * ff * d + 2.0 * n * d + 4.0 * n * d, 6.0 * n * top * ff * d)
        act = torch.empty(n, dense_ff, dtype=bf, device=dev)
        o = torch.empty(n, d, dtype=torch.float32, device=dev)

        def dense():
            if not tc_gemm.gemm_swiglu(h, wgu, act):
                K.swiglu(K.Partials(tc_gemm.partials(h, wgu)), act)
            tc_gemm.gemm(act, wdn, None, o)
        ms = timer(dense)
        note(f"dense_swiglu_{label}", ms, 2.0 * 3 * dense_ff * d + 6.0 * n * d, 6.0 * n * dense_ff * d)
        up, down = Linear(wup), Linear(wdown)
        a2 = torch.empty(n, z["dense"], dtype=bf, device=dev)

        def relu2():
            L.relu2(up.forward(h, defer=True), a2)
            r = down.forward(a2, defer=True, residual=True)
            if isinstance(r, K.Partials):
                r.materialize(torch.float32)
        ms = timer(relu2)
        note(f"dense_relu2_{label}", ms, 2.0 * 2 * z["dense"] * d + 6.0 * n * d, 4.0 * n * z["dense"] * d)

    # ---- the residual: one pass over S streams beside add + RMSNorm over one -------------------------------------------
    for label, n in (("prefill", T), ("decode", batch)):
        xs, yv = rnd(n, S, d, dtype=torch.float32), rnd(n, d, dtype=torch.float32)
        mix, wo, wi = rnd(S, S, dtype=torch.float32), rnd(S, dtype=torch.float32), rnd(S, dtype=torch.float32)
        nw, hb = torch.ones(d, device=dev), torch.empty(n, d, dtype=bf, device=dev)
        ms = timer(lambda: L.hyper_step(xs, yv, mix, wo, wi, nw, 1e-5, hb))
        note(f"hyper_step_{label}", ms, n * d * (8.0 * S + 4 + 2))
        x = rnd(n, d, dtype=torch.float32)
        ms = timer(lambda: K.add_rmsnorm(x, yv, nw, 1e-5, hb))
        note(f"add_rmsnorm_{label}", ms, n * d * (4 + 4 + 4 + 2))
    return rows


def time_banelix_kernels(z, T, context, batch, timer, peaks):
    """Banelix's kernels alone, each beside the kernel of the built-in decoder that does the like job."""
    import numpy as np
    import torch
    from infero_b200 import kernels as K
    from infero_b200.kernels import attention as A, layer_ops as L
    dev, bf = "cuda:0", torch.bfloat16
    d, H, G, D, W, C, nb, taps = z["width"], z["heads"], z["kv"], z["dim"], z["window"], z["rec"], z["blocks"], z["taps"]
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, dtype=bf, k=1.0: (torch.randn(s, generator=g, device=dev) * k).to(dtype)     # noqa: E731
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=dev)                 # noqa: E731
    hbm, tfl = peaks["hbm_gbs"], peaks["bf16_tflops"]
    rows = {}

    def note(name, ms, bytes_=0.0, flops=0.0, **more):
        r = {"us": round(ms * 1e3, 1)}
        if bytes_:
            r["gb_s"] = round(bytes_ / ms / 1e6, 1)
            r["hbm_frac"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["tensor_frac"] = round(flops / ms / 1e9 / tfl, 3)
        r.update(more)
        rows[name] = r

    def batch_ctx(q_lens, pos0, ps=16):
        E_ = len(q_lens)
        per = [-(-(p + n) // ps) for p, n in zip(pos0, q_lens)]
        table = torch.full((E_, max(per)), -1, dtype=torch.int32)
        at = 0
        for e, n in enumerate(per):
            table[e, :n] = torch.arange(at, at + n, dtype=torch.int32)
            at += n
        qs = np.concatenate([[0], np.cumsum(q_lens)[:-1]])
        ctx = types.SimpleNamespace(
            n_entries=E_, n_tokens=int(sum(q_lens)), h_q_len=np.asarray(q_lens, dtype=np.int32), h_pos0=np.asarray(pos0, dtype=np.int32),
            tok_entry=i32(np.repeat(np.arange(E_), q_lens)), positions=i32(np.concatenate([p + np.arange(n) for p, n in zip(pos0, q_lens)])),
            entry_q_start=i32(qs), entry_q_len=i32(q_lens), entry_pos0=i32(pos0), entry_slot=i32(np.arange(E_)), kv_bound=None)
        return ctx, table.to(dev), at

    for label, q_lens, pos0 in (("prefill", [T], [0]), ("decode", [1] * batch, [context - 1] * batch)):
        ctx, table, pages = batch_ctx(q_lens, pos0)
        n = ctx.n_tokens
        # ---- attention: a window and a sink beside all keys and none -----------------------------------------------
        kc, vc = rnd(pages, G, 16, D), rnd(pages, G, 16, D)
        q, out = rnd(n, H * D), torch.empty(n, H * D, dtype=bf, device=dev)
        w = min(W, T if label == "prefill" else context)
        pairs_all = T * T / 2 if label == "prefill" else batch * context
        pairs_win = (T * w - w * w / 2) if label == "prefill" else batch * w
        keys_all = T if label == "prefill" else batch * context
        keys_win = T if label == "prefill" else batch * w
        for name, window, sink, pairs, keys in (("window_sink_attention", W, True, pairs_win, keys_win),
                                                ("gqa_attention", None, False, pairs_all, keys_all)):
            ms = timer(lambda: A.attention_any(q, out, kc, vc, table, ctx.tok_entry, ctx.positions, H, G, D, 16, window, D ** -0.5,
                                               ctx.h_q_len, ctx.h_pos0, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_pos0, sink=sink))
            note(f"{name}_{label}", ms, 2.0 * G * 2 * D * keys + 4.0 * n * H * D, 2.0 * H * 2 * D * pairs)
        # ---- from the input product to queries and the cache: both norms beside rotary + cache append ---------------------
        width = (H + 2 * G) * D
        proj = rnd(n, width, dtype=torch.float32)
        qo = torch.empty(n, H * D, dtype=bf, device=dev)
        fr = torch.rand(D // 2, device=dev, dtype=torch.float64)
        qw, kw = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev)
        ms = timer(lambda: L.qk_prepare(proj, 0, H * D, (H + G) * D, 1, qw, kw, 1e-5, fr, 1.1, ctx.positions, ctx.tok_entry, table,
                                        16, qo, kc, vc, H, G, D, D))
        note(f"qk_prepare_projection_norm_{label}", ms, n * width * (4.0 + 2.0))
        ms = timer(lambda: L.qk_prepare(proj, 0, H * D, -1, 2, None, None, 1e-5, fr, 1.0, ctx.positions, ctx.tok_entry, table,
                                        16, qo, kc, vc, H, G, D, D))
        note(f"qk_prepare_head_norm_{label}", ms, n * (H + G) * D * 4.0 + n * (H + 2 * G) * D * 2.0)
        qkv = rnd(n, width)
        inv = torch.rand(D // 2, device=dev)
        ms = timer(lambda: K.rope_cache(qkv, ctx.positions, ctx.tok_entry, table, inv, kc, vc, H, G, D, 16))
        note(f"rope_cache_{label}", ms, n * width * 2 * 2)
        # ---- the gate per head ---------------------------------------------------------------------------------------
        gate = rnd(n, H, dtype=torch.float32)
        ms = timer(lambda: L.head_gate(out, gate, out, H, D, 0.7))
        note(f"head_gate_{label}", ms, n * H * D * 4.0 + n * H * 4.0)
        # ---- the recurrence: convolution, gate products and scan ------------------------------------------------------
        rctx, _, _ = batch_ctx(q_lens, [0] * len(q_lens))
        bs = C // nb
        yx = rnd(n, 2 * C, dtype=torch.float32)
        cw, cb = rnd(C, taps, dtype=torch.float32, k=0.3), rnd(C, dtype=torch.float32, k=0.1)
        cwt = cw.t().contiguous()
        wg = rnd(nb, 2 * bs, bs, k=bs ** -0.5)
        rb, ib, lam = rnd(C, dtype=torch.float32, k=0.1), rnd(C, dtype=torch.float32, k=0.1), rnd(C, dtype=torch.float32)
        state = torch.zeros(len(q_lens), taps, C, device=dev)
        ro = torch.empty(n, C, dtype=bf, device=dev)
        ms = timer(lambda: L.rglru(yx, 0, C, cw, cb, wg, rb, ib, lam, 8.0, state, rctx.tok_entry, rctx.entry_q_start, rctx.entry_q_len,
                                   rctx.entry_slot, len(q_lens), ro, 0.7, max_q_len=max(q_lens), tensor_cores=True, conv_wt=cwt))
        least = n * C * (8.0 + 2.0) + 2.0 * wg.numel() + 8.0 * len(q_lens) * taps * C
        moved = least + n * C * (4.0 + 2.0 + 4.0 + 8.0 + 8.0 + 4.0)           # u written and read twice (+ bf16), gates written and read
        note(f"rglru_{label}", ms, least, 2.0 * n * 2 * C * bs, gb_s_with_intermediates=round(moved / ms / 1e6, 1),
             hbm_frac_with_intermediates=round(moved / ms / 1e6 / hbm, 3))
        # ---- add + RMSNorm with the sublayer's result times a constant (the same kernel as without) -----------------------
        x, yv = rnd(n, d, dtype=torch.float32), rnd(n, d, dtype=torch.float32)
        nw, hb = torch.ones(d, device=dev), torch.empty(n, d, dtype=bf, device=dev)
        ms = timer(lambda: K.add_rmsnorm(x, yv, nw, 1e-5, hb, delta_scale=0.5))
        note(f"add_rmsnorm_scaled_{label}", ms, n * d * (4 + 4 + 4 + 2))
    return rows


def time_pibavik_kernels(z, T, context, batch, timer, peaks):
    """Pibavik's kernels alone, each beside the kernel of another design that does the like job."""
    import numpy as np
    import torch
    from infero_b200 import kernels as K
    from infero_b200.kernels import attention as A, layer_ops as L, moe as M
    dev, bf = "cuda:0", torch.bfloat16
    d, H, G, D, W = z["width"], z["heads"], z["kv"], z["dim"], z["window"]
    Hn, P, N, Gs, taps, parts = z["ssd_heads"], z["ssd_vdim"], z["state"], z["groups"], z["taps"], z["norm_groups"]
    E, top, ff = z["experts"], z["top"], z["ff"]
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, dtype=bf, k=1.0: (torch.randn(s, generator=g, device=dev) * k).to(dtype)     # noqa: E731
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=dev)                 # noqa: E731
    hbm, tfl = peaks["hbm_gbs"], peaks["bf16_tflops"]
    rows = {}

    def note(name, ms, bytes_=0.0, flops=0.0, **more):
        r = {"us": round(ms * 1e3, 1)}
        if bytes_:
            r["gb_s"] = round(bytes_ / ms / 1e6, 1)
            r["hbm_frac"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["tensor_frac"] = round(flops / ms / 1e9 / tfl, 3)
        r.update(more)
        rows[name] = r

    def batch_ctx(q_lens, pos0, ps=16):
        E_ = len(q_lens)
        per = [-(-(p + n) // ps) for p, n in zip(pos0, q_lens)]
        table = torch.full((E_, max(per)), -1, dtype=torch.int32)
        at = 0
        for e, n in enumerate(per):
            table[e, :n] = torch.arange(at, at + n, dtype=torch.int32)
            at += n
        qs = np.concatenate([[0], np.cumsum(q_lens)[:-1]])
        ctx = types.SimpleNamespace(
            n_entries=E_, n_tokens=int(sum(q_lens)), h_q_len=np.asarray(q_lens, dtype=np.int32), h_pos0=np.asarray(pos0, dtype=np.int32),
            tok_entry=i32(np.repeat(np.arange(E_), q_lens)), positions=i32(np.concatenate([p + np.arange(n) for p, n in zip(pos0, q_lens)])),
            entry_q_start=i32(qs), entry_q_len=i32(q_lens), entry_pos0=i32(pos0), entry_slot=i32(np.arange(E_)), kv_bound=None)
        return ctx, table.to(dev), at

    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float32, device=dev)
    for label, q_lens, pos0 in (("prefill", [T], [0]), ("decode", [1] * batch, [context - 1] * batch)):
        ctx, table, pages = batch_ctx(q_lens, pos0)
        n = ctx.n_tokens
        # ---- window attention with a distance bias beside window attention with a sink -------------------------------
        kc, vc = rnd(pages, G, 16, D), rnd(pages, G, 16, D)
        q, out = rnd(n, H * D), torch.empty(n, H * D, dtype=bf, device=dev)
        w = min(W, T if label == "prefill" else context)
        pairs = (T * w - w * w / 2) if label == "prefill" else batch * w
        keys = T if label == "prefill" else batch * w
        for name, sink, sl in (("window_bias_attention", False, slopes), ("window_sink_attention", True, None)):
            ms = timer(lambda: A.attention_any(q, out, kc, vc, table, ctx.tok_entry, ctx.positions, H, G, D, 16, W, D ** -0.5,
                                               ctx.h_q_len, ctx.h_pos0, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_pos0,
                                               sink=sink, slopes=sl))
            note(f"{name}_{label}", ms, 2.0 * G * 2 * D * keys + 4.0 * n * H * D, 2.0 * H * 2 * D * pairs)
        # ---- from the input product to queries and the cache: the norm per head beside the norm over the projection ------
        width = (H + 2 * G) * D
        proj = rnd(n, width, dtype=torch.float32)
        qo = torch.empty(n, H * D, dtype=bf, device=dev)
        fr = torch.rand(D // 4, device=dev, dtype=torch.float64)
        for name, mode, qw, kw in (("qk_prepare_weighted_head_norm", 3, torch.ones(D, device=dev), torch.ones(D, device=dev)),
                                   ("qk_prepare_projection_norm", 1, torch.ones(H * D, device=dev), torch.ones(G * D, device=dev))):
            ms = timer(lambda: L.qk_prepare(proj, 0, H * D, (H + G) * D, mode, qw, kw, 1e-5, fr, 1.0, ctx.positions, ctx.tok_entry,
                                            table, 16, qo, kc, vc, H, G, D, D))
            note(f"{name}_{label}", ms, n * width * (4.0 + 2.0))
        # ---- the state-space recurrence beside the gated linear recurrence of equal width -----------------------------
        rctx, _, _ = batch_ctx(q_lens, [0] * len(q_lens))
        inner, CH = Hn * P, Hn * P + 2 * Gs * N
        zx = rnd(n, 2 * inner + 2 * Gs * N + Hn, dtype=torch.float32, k=0.5)
        cw, cb = rnd(CH, taps, dtype=torch.float32, k=0.3), rnd(CH, dtype=torch.float32, k=0.1)
        dtb, alog, skip = rnd(Hn, dtype=torch.float32) - 3.0, rnd(Hn, dtype=torch.float32, k=0.2), rnd(Hn, dtype=torch.float32)
        nw = torch.ones(inner, device=dev)
        state = torch.zeros(len(q_lens), L.ssd_state_floats(Hn, N, P, Gs, taps), device=dev)
        so = torch.empty(n, inner, dtype=bf, device=dev)
        ms = timer(lambda: L.ssd(zx, 0, inner, inner + CH, cw, cb, dtb, alog, skip, nw, 1e-5, parts, state, rctx.tok_entry,
                                 rctx.entry_q_start, rctx.entry_q_len, rctx.entry_slot, len(q_lens), so, Hn, Gs, N, P, 0.7,
                                 max_q_len=max(q_lens)))
        least = n * (zx.shape[1] * 4.0 + inner * 2.0) + 8.0 * state.numel()
        moved = least + n * (CH * 8.0 + inner * 8.0)                       # the convolution's result and y written and read
        note(f"ssd_{label}", ms, least, 2.0 * n * Hn * N * P * 2, gb_s_with_intermediates=round(moved / ms / 1e6, 1),
             hbm_frac_with_intermediates=round(moved / ms / 1e6 / hbm, 3))
        C, nb = inner, H
        bs = C // nb
        yx = rnd(n, 2 * C, dtype=torch.float32)
        rw, rb_ = rnd(C, taps, dtype=torch.float32, k=0.3), rnd(C, dtype=torch.float32, k=0.1)
        wg = rnd(nb, 2 * bs, bs, k=bs ** -0.5)
        rb, ib, lam = rnd(C, dtype=torch.float32, k=0.1), rnd(C, dtype=torch.float32, k=0.1), rnd(C, dtype=torch.float32)
        rstate = torch.zeros(len(q_lens), taps, C, device=dev)
        ro = torch.empty(n, C, dtype=bf, device=dev)
        ms = timer(lambda: L.rglru(yx, 0, C, rw, rb_, wg, rb, ib, lam, 8.0, rstate, rctx.tok_entry, rctx.entry_q_start, rctx.entry_q_len,
                                   rctx.entry_slot, len(q_lens), ro, 0.7, max_q_len=max(q_lens), tensor_cores=True))
        note(f"rglru_{label}", ms, n * C * (8.0 + 2.0) + 2.0 * wg.numel() + 8.0 * len(q_lens) * taps * C, 2.0 * n * 2 * C * bs)
        # ---- ungated experts that read their weighted input beside gated experts of the same sizes --------------------
        h = rnd(n, d)
        up, down = rnd(E, ff, d, k=d ** -0.5), rnd(E, d, ff, k=ff ** -0.5)
        gate_up = rnd(E, 2 * ff, d, k=d ** -0.5)
        logits = rnd(n, E, dtype=torch.float32)
        idx, wts = L.moe_select_scored(logits, E, top)
        y = torch.empty(n, d, dtype=torch.float32, device=dev)
        touched = min(E, n * top)
        ms = timer(lambda: M.plain_experts(h, up, down, idx, wts, True, None, y))
        note(f"experts_relu2_weighted_input_{label}", ms, touched * 2.0 * ff * d * 2 + n * d * (2.0 + 4.0), 2.0 * n * top * 2 * ff * d)
        ms = timer(lambda: M.experts(h, gate_up, down, idx, wts, None, None, y))
        note(f"experts_swiglu_{label}", ms, touched * 3.0 * ff * d * 2 + n * d * (2.0 + 4.0), 2.0 * n * top * 3 * ff * d)
        ms = timer(lambda: L.moe_select_scored(logits, E, top))
        note(f"select_by_sigmoid_scores_{label}", ms, n * E * 4.0 + n * top * 8.0)
        ms = timer(lambda: L.moe_select(logits, E, top))
        note(f"select_by_softmax_of_chosen_{label}", ms, n * E * 4.0 + n * top * 8.0)
        # ---- the norm of a column slice (the queries' latent) beside add + RMSNorm ------------------------------------
        Q = z["q_rank"]
        wide = rnd(n, Q + z["kv_rank"], dtype=torch.float32)
        cq = torch.empty(n, Q, dtype=bf, device=dev)
        qn = torch.ones(Q, device=dev)
        ms = timer(lambda: L.gated_group_norm(wide[:, :Q], None, qn, 1e-5, 1, cq))
        note(f"latent_query_norm_{label}", ms, n * Q * (4.0 + 2.0))
        x, yv = rnd(n, d, dtype=torch.float32), rnd(n, d, dtype=torch.float32)
        nw2, hb = torch.ones(d, device=dev), torch.empty(n, d, dtype=bf, device=dev)
        ms = timer(lambda: K.add_rmsnorm(x, yv, nw2, 1e-5, hb))
        note(f"add_rmsnorm_{label}", ms, n * d * (4 + 4 + 4 + 2))
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="design_bench")
    ap.add_argument("--design", default="vufizen", choices=["vufizen", "gositar", "banelix", "pibavik"])
    ap.add_argument("--sizes", default="s,m")
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--kernels-at", default="m", help="the size whose kernels are timed alone ('' for none)")
    args = ap.parse_args(argv)
    import torch
    from infero_b200 import kernels as K
    K.lib()
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        peaks = {"hbm_gbs": float(m["hbm_gbs"]), "bf16_tflops": float(m["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        pass
    timer = _Timer()
    sizes, design_cfg, beside_cfg, each = {"vufizen": (SIZES, vufizen_config, qwen2_config, time_kernels),
                                           "gositar": (GOSITAR_SIZES, gositar_config, qwen2_beside_gositar, time_gositar_kernels),
                                           "banelix": (BANELIX_SIZES, banelix_config, qwen2_beside_banelix, time_banelix_kernels),
                                           "pibavik": (PIBAVIK_SIZES, pibavik_config, banelix_beside_pibavik, time_pibavik_kernels)}[args.design]
    beside = "banelix" if args.design == "pibavik" else "qwen2"
    out = {"bench": "designs", "design": args.design, "dtype": "bf16", "data": "synthetic", "prompt": args.prompt, "context": args.context,
           "batch": args.batch, "layers": args.layers, "peaks": peaks, "sizes": {}}
    for name in [s for s in args.sizes.split(",") if s]:
        z = sizes[name]
        out["sizes"][name] = {"shape": z,
                              args.design: time_model(design_cfg(z, args.layers), args.prompt, args.context, args.batch, timer),
                              beside: time_model(beside_cfg(z, args.layers), args.prompt, args.context, args.batch, timer)}
        print(f"[design_bench] {name}: {json.dumps(out['sizes'][name])}", file=sys.stderr, flush=True)
    if args.kernels_at:
        out["kernels"] = {"size": args.kernels_at,
                          "rows": each(sizes[args.kernels_at], args.prompt, args.context, args.batch, timer, peaks)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
