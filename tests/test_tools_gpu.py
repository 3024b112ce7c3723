"""The measurement tools run: the timeline of a decode step (the library's timeline variant, every block's
first and last nanosecond) and one kernel alone."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args):
    env = dict(os.environ, PYTHONPATH=ROOT)
    env.pop("INFERO_TIMELINE", None)
    r = subprocess.run([sys.executable, "-m"] + args, capture_output=True, text=True, cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


def test_timeline_of_a_decode_step():
    """The averaged layer of a step of single tokens: its launches in the order they started, decode
    attention among them, and launches seen to start before the one in front has ended (programmatic
    dependent launch)."""
    out = _run(["infero_b200.tools.timeline", "--batch", "2", "--context", "300", "--layers", "6", "--shape", "0.5b"])
    assert "decode attention" in out and "a layer every" in out, out[-1500:]
    rows = [ln.split() for ln in out.splitlines() if ln.startswith(("product", "decode attention", "norm"))]
    assert len(rows) >= 5
    # the table of the averaged layer: columns are name..., blocks, SMs, first start, all started, first end, last end, busy
    layer = []
    for ln in out.splitlines():
        if ln.startswith("a layer every"):
            break
        if ln.startswith(("product", "decode attention", "norm", "swiglu", "rotary")):
            layer.append(ln)
    assert any(ln.startswith("decode attention") for ln in layer)
    firsts = [float(ln.split()[-5]) for ln in layer]
    ends = [float(ln.split()[-2]) for ln in layer]
    assert all(b >= a for a, b in zip(firsts, firsts[1:])), "launches are listed in the order they started"
    assert any(firsts[i + 1] < ends[i] for i in range(len(layer) - 1)), "no launch started under the one in front"


def test_one_kernel_alone():
    out = _run(["infero_b200.tools.kernel_bench", "attn_decode_fused", "--batch", "2", "--context", "512", "--reps", "3"])
    assert "attn_decode_fused:" in out and "us per launch" in out and "error flag" not in out


def test_design_bench_prints_both_designs_and_the_kernels(capsys):
    """``bench.py --designs`` at a size made for tests: both models step, every kernel row has a time."""
    import json
    from infero_b200.tools import design_bench
    assert design_bench.main(["--sizes", "t", "--prompt", "600", "--context", "300", "--batch", "3", "--layers", "2",
                              "--kernels-at", "t"]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["bench"] == "designs" and set(line["sizes"]["t"]) == {"shape", "vufizen", "qwen2"}
    for design in ("vufizen", "qwen2"):
        assert line["sizes"]["t"][design]["prefill_tok_s"] > 0 and line["sizes"]["t"][design]["decode_tok_s"] > 0
    rows = line["kernels"]["rows"]
    assert {"diff_attention_prefill", "hgrn2_scan_prefill", "moe_experts_decode", "gated_norm_add_prefill"} <= set(rows)
    assert all(r["us"] > 0 for r in rows.values())


def test_design_bench_of_gositar(capsys):
    """``bench.py --designs --design gositar`` at a size made for tests."""
    import json
    from infero_b200.tools import design_bench
    assert design_bench.main(["--design", "gositar", "--sizes", "t", "--prompt", "600", "--context", "300", "--batch", "3",
                              "--layers", "2", "--kernels-at", "t"]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["design"] == "gositar" and set(line["sizes"]["t"]) == {"shape", "gositar", "qwen2"}
    for design in ("gositar", "qwen2"):
        assert line["sizes"]["t"][design]["prefill_tok_s"] > 0 and line["sizes"]["t"][design]["decode_tok_s"] > 0
    rows = line["kernels"]["rows"]
    assert {"latent_attention_prefill", "latent_attention_decode", "moe_experts_clamped_decode", "hyper_step_prefill",
            "per_head_up_k_prefill", "dense_relu2_decode"} <= set(rows)
    assert all(r["us"] > 0 for r in rows.values())


def test_design_bench_of_pibavik(capsys):
    """``bench.py --designs --design pibavik`` at a size made for tests: beside Banelix, the closest design."""
    import json
    from infero_b200.tools import design_bench
    assert design_bench.main(["--design", "pibavik", "--sizes", "t", "--prompt", "600", "--context", "300", "--batch", "3",
                              "--layers", "4", "--kernels-at", "t"]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["design"] == "pibavik" and set(line["sizes"]["t"]) == {"shape", "pibavik", "banelix"}
    for design in ("pibavik", "banelix"):
        assert line["sizes"]["t"][design]["prefill_tok_s"] > 0 and line["sizes"]["t"][design]["decode_tok_s"] > 0
    rows = line["kernels"]["rows"]
    assert {"window_bias_attention_prefill", "window_bias_attention_decode", "ssd_prefill", "ssd_decode", "rglru_decode",
            "experts_relu2_weighted_input_prefill", "experts_swiglu_decode", "latent_query_norm_prefill"} <= set(rows)
    assert all(r["us"] > 0 for r in rows.values())
