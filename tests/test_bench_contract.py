"""CPU checks of bench.py: the algorithmic work that roofline figures are computed from, and the JSON
line of the reference arm (the oracle port timed on the host cores)."""

import importlib.util
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_work_per_step():
    """18*R*H*I FLOP for the six grouped GEMMs of a step, and the byte counts of the row movers: the figures
    quoted for the benchmark configurations (TFLOP / GB per step and GPU)."""
    bench = _bench()
    want_tflop = {"mixtral_c3": 34.63, "finegrained_c4": 7.42, "ep_c5": 59.37, "small_c1": 0.0773}
    for name, tflop in want_tflop.items():
        work = bench.algorithmic_work(bench.WORKLOADS[name])
        assert abs(work["gemm_flops_total"] / 1e12 - tflop) < 0.01 * tflop, name
        # per entry point: bf16 runs the two SwiGLU-fused GEMMs, fp32 runs plain forward/dgrad twice instead
        fused = ("fma_b200_moe_gemm_forward_swiglu", "fma_b200_moe_gemm_dgrad_swiglu")
        used = [v for k, v in work["gemm_flops"].items() if bench.WORKLOADS[name]["dtype"] == "bf16" or k not in fused]
        assert sum(used) == work["gemm_flops_total"], name
    c5 = bench.algorithmic_work(bench.WORKLOADS["ep_c5"])["hbm_bytes"]
    assert abs(c5["fma_b200_moe_scatter"] / 1e9 - 4.836) < 0.005
    assert abs(c5["fma_b200_moe_combine"] / 1e9 - 4.833) < 0.005
    c3 = bench.algorithmic_work(bench.WORKLOADS["mixtral_c3"])["hbm_bytes"]
    assert abs(c3["fma_b200_moe_scatter"] / 1e9 - 0.403) < 0.001


def test_cpu_sample_is_bounded():
    bench = _bench()
    for cfg in bench.WORKLOADS.values():
        experts, toks = bench.cpu_sample(cfg)
        assert 1 <= toks <= cfg["T"] and 1 <= experts <= cfg["E"]
        assert experts == cfg["E"] or experts == cfg["k"]  # the whole workload, or k experts that every token visits
        assert 18 * cfg["k"] * cfg["H"] * cfg["I"] * toks <= bench.CPU_SAMPLE_FLOPS or toks == 64
        assert toks <= max(64, cfg["T"] * cfg["k"] // cfg["E"]) or experts == cfg["E"]  # never more rows per expert than the workload gives
        assert bench.cpu_sample_text(cfg)


def test_reference_arm_json_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "small_c1",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, check=True)  # fmt: skip
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "moe_layer_fwd_bwd_tokens_per_s"
    for key in ("value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "cpu_baseline", "e2e"):  # fmt: skip
        assert key in line, key
    assert line["vs_baseline"] is None and line["higher_is_better"] is True and line["config"]["workload"] == "small_c1"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["value"] == line["value"]
    assert line["cpu_baseline"]["cores"] >= 1 and line["cpu_baseline"]["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
