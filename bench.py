"""Benchmark of the MoE-layer hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE for N > 1).  A step is one forward +
backward of the layer over one batch of seeded synthetic tokens.  Rank 0 prints ONE JSON line.

Workloads (all synthetic, shapes from the benchmark specification):
  ep_c5          per GPU T=65536, H=4096, E=128 experts in total sharded over the N ranks, top-8,
                 I=1536, bf16, uniform router.  Default at every N (at N=1 all 128 experts are local),
                 so the 1/2/4/8-GPU series is one weak-scaling series.
  mixtral_c3     T=16384, H=4096, E=8, top-2, I=14336, bf16 (single GPU)
  finegrained_c4 T=32768, H=2048, E=128, top-8, I=768, bf16, Zipf(1.0) expert load (single GPU)
  small_c1       T=4096, H=1024, E=8, top-2, I=512, fp32 (single GPU)
  count_c2       continuous_count alone: 2^24 int32 ids, 128 bins, uniform or Zipf(1.1)

Keys of the JSON line beyond the common ones:
  value      tokens/s of the whole job with inputs resident in HBM (device-timed, max over ranks)
  e2e        the same through the public API with HOST (pinned) x and dy: H2D copies of both and D2H
             copies of y and dx are inside the timed region
  roofline   for the dominant kernel (the tcgen05 grouped GEMMs: all six launches of a step), achieved
             TFLOP/s from CUDA events around the launches inside the timed region
  kernels    per entry point: calls per step, ms per step, achieved GB/s or TFLOP/s, fraction of peak
  cpu_baseline  the CPU oracle (numpy port of the reference's torch backend) timed on this host on a
             bounded sample of the same workload (N=1, rank 0 only)

`--impl reference` times that CPU port on the same workload description instead of the CUDA path.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT / "cute-kernels_b200", ROOT):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import numpy as np  # noqa: E402
import torch  # noqa: E402

WORKLOADS = {
    "ep_c5": dict(T=65536, H=4096, E=128, k=8, I=1536, dtype="bf16", router="uniform"),
    "mixtral_c3": dict(T=16384, H=4096, E=8, k=2, I=14336, dtype="bf16", router="uniform"),
    "finegrained_c4": dict(T=32768, H=2048, E=128, k=8, I=768, dtype="bf16", router="zipf"),
    "small_c1": dict(T=4096, H=1024, E=8, k=2, I=512, dtype="f32", router="uniform"),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=self.file, stderr=subprocess.DEVNULL)  # fmt: skip
        except Exception:
            self.proc = None

    def stop(self) -> dict | None:
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        rows = [line.split(", ") for line in Path(self.file.name).read_text().strip().splitlines() if line.strip()]
        os.unlink(self.file.name)
        rows = [r for r in rows if len(r) >= 9]
        if not rows:
            return None
        sm = sorted(float(r[1]) for r in rows)
        reasons = set()
        for r in rows:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][2]), "reasons": sorted(reasons),
                "samples": len(rows), "power_w_max": max(float(r[3]) for r in rows)}  # fmt: skip


# ---------------------------------------------------------------------------------------------
# synthetic data
# ---------------------------------------------------------------------------------------------
def make_layer(cfg: dict, rank: int, world: int, device: torch.device):
    """The layer with seeded N(0, 0.02) weights.  Expert e is drawn from seed 1000+e, so a sharded run
    holds exactly the experts of the unsharded one."""
    import fma_b200

    dtype = torch.bfloat16 if cfg["dtype"] == "bf16" else torch.float32
    E, k, H, I = cfg["E"], cfg["k"], cfg["H"], cfg["I"]
    with torch.device("meta"):
        cls = fma_b200.ExpertParallelMoE if world > 1 else fma_b200.MoE
        layer = cls(E, k, H, I, fma_b200.swiglu_packed, True, False, 0.02)
    layer = layer.to_empty(device=device).to(dtype)
    gen = torch.Generator(device=device)
    first = rank * (E // world) if world > 1 else 0
    with torch.no_grad():
        for j in range(layer.c_fc.weight.size(0)):
            gen.manual_seed(1000 + first + j)
            layer.c_fc.weight[j].copy_(torch.randn(layer.c_fc.weight.shape[1:], generator=gen, device=device) * 0.02)
            layer.c_proj.weight[j].copy_(torch.randn(layer.c_proj.weight.shape[1:], generator=gen, device=device) * 0.02)
        gen.manual_seed(7)
        layer.gate.weight.copy_(torch.randn(E, H, generator=gen, device=device) * 0.02)
        for m in (layer.c_fc, layer.c_proj):
            m.N_array.fill_(m.out_features)
            m.K_array.fill_(m.in_features)
        if cfg["router"] == "zipf":
            # per-expert bias so that expert load follows Zipf(1.0) over a seeded permutation
            gate = torch.nn.Linear(H, E, bias=True, device=device, dtype=dtype)
            p = 1.0 / torch.arange(1, E + 1, dtype=torch.float64)
            perm = torch.randperm(E, generator=torch.Generator().manual_seed(3))
            gate.weight.copy_(layer.gate.weight)
            gate.bias.copy_(torch.log(p / p.sum())[perm].to(dtype))
            layer.gate = gate
    return layer, dtype


def make_inputs(cfg: dict, rank: int, device: torch.device, dtype):
    gen = torch.Generator(device=device)
    gen.manual_seed(100 + rank)
    x = torch.randn(cfg["T"], cfg["H"], generator=gen, device=device).to(dtype)
    dy = torch.randn(cfg["T"], cfg["H"], generator=gen, device=device).to(dtype)
    return x, dy


def layer_step(layer, x, dy):
    for p in layer.parameters():
        p.grad = None
    x.grad = None
    y, _ = layer(x)
    y.backward(dy)
    return y


def write_timeline(path: str, step, rank: int, barrier) -> None:
    """One step under torch.profiler (kineto) on rank 0, the other ranks run it plainly; the file lists
    every device activity in start order.  Shows what overlaps what (GEMMs, exchanges, waits); durations
    under the profiler are not benchmark numbers."""
    barrier()
    if rank != 0:
        step()
        barrier()
        return
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize()
    with tempfile.TemporaryDirectory() as tmp:
        raw = os.path.join(tmp, "trace.json")
        prof.export_chrome_trace(raw)
        with open(raw) as f:
            events = json.load(f)["traceEvents"]
    acts = sorted((e for e in events if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset")), key=lambda e: e["ts"])
    t0 = acts[0]["ts"] if acts else 0
    with open(path, "w") as f:
        f.write("# start_ms duration_ms stream name\n")
        for e in acts:
            f.write("%9.3f %8.3f s%-3s %s\n" % ((e["ts"] - t0) / 1e3, e["dur"] / 1e3, e["args"].get("stream", "?"),
                                               e["name"][:90]))  # fmt: skip
    barrier()


# ---------------------------------------------------------------------------------------------
# algorithmic work (what roofline figures are computed from)
# ---------------------------------------------------------------------------------------------
def algorithmic_work(cfg: dict) -> dict:
    T, H, E, k, I = cfg["T"], cfg["H"], cfg["E"], cfg["k"], cfg["I"]
    s = 2 if cfg["dtype"] == "bf16" else 4
    R = T * k
    gemm = {  # FLOPs = 2*M*N*K over token rows only (no padding counted)
        "fma_b200_moe_gemm_forward_swiglu": 4 * R * H * I,
        "fma_b200_moe_gemm_forward": 2 * R * H * I + (4 * R * H * I if cfg["dtype"] == "f32" else 0),
        "fma_b200_moe_gemm_dgrad_swiglu": 2 * R * H * I,
        "fma_b200_moe_gemm_dgrad": 4 * R * H * I + (2 * R * H * I if cfg["dtype"] == "f32" else 0),
        "fma_b200_moe_gemm_wgrad": 6 * R * H * I,
    }
    hbm = {  # bytes
        "fma_b200_moe_scatter": (T + R) * H * s + R * 8,
        "fma_b200_moe_combine": (R + T) * H * s + R * s,
        "fma_b200_moe_combine_backward": (T + 2 * R) * H * s + R * s,
        "fma_b200_moe_scatter_backward": (R + T) * H * s,
        "fma_b200_moe_sort": 2 * R * 8 + 2 * R * 4,
        "fma_b200_router_topk_softmax": T * E * s + T * k * (s + 8),
        "fma_b200_router_topk_softmax_backward": T * E * s + T * k * (2 * s + 8),
    }
    return {"gemm_flops": gemm, "hbm_bytes": hbm, "gemm_flops_total": 18 * R * H * I}


# ---------------------------------------------------------------------------------------------
# CPU baseline (the oracle port), bounded sample
# ---------------------------------------------------------------------------------------------
CPU_SAMPLE_FLOPS = 0.6e12  # expert-GEMM work of one CPU pass (forward + backward)


def cpu_sample(cfg: dict) -> tuple[int, int]:
    """(experts, tokens) of the bounded CPU sample.  The sample keeps what decides the cost per token: the
    per-expert problem.  It takes k of the E experts and routes every sampled token to all k of them, so each
    expert sees as many rows as tokens are sampled; the token count is what the full workload gives an expert
    (T*k/E rows under uniform routing), capped so that one pass stays near CPU_SAMPLE_FLOPS.  (A sample of few
    tokens over ALL experts would time weight-sized work - reading and rounding every expert's weights and
    weight gradients - that the full workload amortises over thousands of rows per expert.)"""
    if 18 * cfg["T"] * cfg["k"] * cfg["H"] * cfg["I"] <= CPU_SAMPLE_FLOPS:
        return cfg["E"], cfg["T"]  # the whole workload is small enough: all experts, real top-k routing
    e_s = min(cfg["E"], cfg["k"])
    full_load = max(1, cfg["T"] * cfg["k"] // cfg["E"])
    budget = int(CPU_SAMPLE_FLOPS / (18 * cfg["k"] * cfg["H"] * cfg["I"]))
    return e_s, max(64, min(full_load, budget, cfg["T"]))


def cpu_oracle_pass(cfg: dict, weights: dict, seed: int, tokens: int = 0) -> tuple[float, int]:
    """One forward+backward of the oracle on a seeded sample; returns (seconds, tokens).  `weights` holds the
    sampled experts (cpu_sample(cfg)[0] of them); `tokens` overrides the sample's token count (warm-up)."""
    from oracle import moe_oracle as O

    e_s = weights["w_fc"].shape[0]
    t_s = tokens or cpu_sample(cfg)[1]
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((t_s, cfg["H"]), dtype=np.float32)
    dy = rng.standard_normal((t_s, cfg["H"]), dtype=np.float32)
    if cfg["dtype"] == "bf16":
        x, dy = O.bf16_round(x), O.bf16_round(dy)
    t0 = time.perf_counter()
    fwd = O.moe_forward(x, weights["w_gate"][:e_s], weights["w_fc"][:e_s], weights["w_proj"][:e_s], min(cfg["k"], e_s),
                        cfg["dtype"])  # fmt: skip
    O.moe_backward(fwd, dy, keep_weight_grads=False)
    return time.perf_counter() - t0, t_s


def cpu_sample_text(cfg: dict) -> str:
    e_s, t_s = cpu_sample(cfg)
    if e_s == cfg["E"]:
        return (f"the whole workload ({t_s} tokens, top-{cfg['k']} of {e_s} experts), numpy fp32 matmul with "
                f"{cfg['dtype']} rounding points")
    return (f"{t_s} tokens, each routed to the same {e_s} of the {cfg['E']} experts ({t_s} rows per expert; the full "
            f"workload gives an expert {cfg['T'] * cfg['k'] // cfg['E']}), numpy fp32 matmul with {cfg['dtype']} "
            f"rounding points")


def host_weights_from_layer(layer, n_experts: int) -> dict:
    """The router weight and the first n_experts experts of the layer, as float32 host arrays."""
    f = lambda t: t.detach().float().cpu().numpy()  # noqa: E731
    return {"w_gate": f(layer.gate.weight[:n_experts]), "w_fc": f(layer.c_fc.weight[:n_experts]),
            "w_proj": f(layer.c_proj.weight[:n_experts])}  # fmt: skip


def host_weights_seeded(cfg: dict) -> dict:
    """Weights of the sampled experts for the reference arm: seeded N(0, 0.02), bf16-rounded if needed."""
    from oracle import moe_oracle as O

    rng = np.random.default_rng(1000)
    E, H, I = cpu_sample(cfg)[0], cfg["H"], cfg["I"]
    w = {"w_gate": rng.standard_normal((E, H), dtype=np.float32) * 0.02,
         "w_fc": rng.standard_normal((E, 2 * I, H), dtype=np.float32) * 0.02,
         "w_proj": rng.standard_normal((E, H, I), dtype=np.float32) * 0.02}  # fmt: skip
    if cfg["dtype"] == "bf16":
        w = {n: O.bf16_round(a) for n, a in w.items()}
    return w


CPU_THREADS_MAX = 16


def pin_cpu_threads() -> int:
    """Sets the BLAS thread count of the CPU arm itself - min(host cores, 16) - so that it does not depend on
    what the launcher exported (torchrun sets OMP_NUM_THREADS=1); returns the count in effect."""
    want = max(1, min(os.cpu_count() or 1, CPU_THREADS_MAX))
    try:
        from threadpoolctl import threadpool_info, threadpool_limits

        threadpool_limits(limits=want, user_api="blas")
        n = [p.get("num_threads", 1) for p in threadpool_info() if p.get("user_api") == "blas"]
        if n:
            return int(max(n))
    except Exception:
        pass
    return 1


# ---------------------------------------------------------------------------------------------
# reference arm
# ---------------------------------------------------------------------------------------------
def run_reference(args, cfg: dict, name: str) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = pin_cpu_threads()
    weights = host_weights_seeded(cfg)
    for i in range(args.warmup):
        cpu_oracle_pass(cfg, weights, seed=i)
    secs, toks = 0.0, 0
    for i in range(args.steps):
        s, t = cpu_oracle_pass(cfg, weights, seed=100 + i)
        secs += s
        toks += t
    value = toks / secs
    line = {
        "impl": "reference", "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * secs / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic",
        "config": {"workload": name, **{k: cfg[k] for k in ("T", "H", "E", "k", "I")},
                   "note": "CPU port of the reference torch backend; each step is a bounded sample of the workload"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": "per step: " + cpu_sample_text(cfg)},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# continuous_count workload
# ---------------------------------------------------------------------------------------------
def measure_count(peaks: dict, steps: int, warmup: int, variants=(0,), big: bool = True) -> tuple[dict, float]:
    """continuous_count on 2^24 int32 ids in 128 bins, uniform and Zipf(1.1): {case: ms, GB/s, fraction of the
    HBM peak} and the CPU time of torch.bincount on the same ids (ms)."""
    import fma_b200

    dev = torch.device("cuda:0")
    n, E = 1 << 24, 128
    sys.path.insert(0, str(ROOT / "tests"))
    from _util import zipf_ids

    results = {}
    n_copies = 8  # 8 x 64 MB of ids, visited round-robin: every launch reads data that is not in the 126 MB L2
    for dist_name, ids in (("uniform", torch.randint(0, E, (n,), dtype=torch.int32, generator=torch.Generator().manual_seed(0))),
                           ("zipf1.1", zipf_ids(n, E, 1.1, seed=1))):
        ref = torch.bincount(ids.long(), minlength=E)
        copies = [ids.to(dev) for _ in range(n_copies)]
        for variant in variants:
            out = fma_b200.continuous_count(copies[0], E, _variant=variant)
            assert torch.equal(out.to(torch.int64).cpu(), ref)
            times = []
            for i in range(warmup + steps):
                torch.cuda._sleep(400_000)  # keep the GPU busy while the timed launch is enqueued (no host gap in the interval)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fma_b200.continuous_count(copies[i % n_copies], E, _variant=variant)
                b.record()
                torch.cuda.synchronize()
                if i >= warmup:
                    times.append(a.elapsed_time(b))
            ms = float(np.median(times))
            gbs = (n * 4 + E * 4) / ms / 1e6
            results[f"{dist_name}/variant{variant}"] = {"ms": ms, "gbs": gbs, "frac": gbs / peaks["hbm_gbs"]}
        if dist_name == "uniform":
            # Floors of this measurement, timed the same way (events around one launch behind a busy GPU): a
            # library copy of the same 64 MB into a resident buffer (reads AND writes 64 MB), and a kernel that
            # does nothing (what the two event records and the launch cost by themselves).
            scratch = torch.empty_like(copies[0])
            for label, fn in (("copy_64MB", lambda i: scratch.copy_(copies[i % n_copies])),
                              ("empty_launch", lambda i: torch.cuda._sleep(1))):
                times = []
                for i in range(warmup + steps):
                    torch.cuda._sleep(400_000)
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    fn(i)
                    b.record()
                    torch.cuda.synchronize()
                    if i >= warmup:
                        times.append(a.elapsed_time(b))
                ms = float(np.median(times))
                results[f"floor/{label}"] = {"ms": ms}
        del copies
    if big:
        # streaming rate on an input 16x larger (1 GiB of ids), default variant: shows the size-independent part
        big_ids = torch.randint(0, E, (n * 16,), dtype=torch.int32, device=dev)
        times = []
        for i in range(8):
            torch.cuda._sleep(400_000)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fma_b200.continuous_count(big_ids, E)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        big_ms = float(np.median(times[3:]))
        results["uniform_2^28_ids/default"] = {"ms": big_ms, "gbs": n * 16 * 4 / big_ms / 1e6,
                                               "frac": n * 16 * 4 / big_ms / 1e6 / peaks["hbm_gbs"]}
        del big_ids
    t0 = time.perf_counter()
    for _ in range(3):
        torch.bincount(ids.long(), minlength=E)
    cpu_ms = (time.perf_counter() - t0) / 3 * 1e3
    return results, cpu_ms


def run_count(args, peaks, peaks_kind) -> None:
    from fma_b200 import _native

    n, E = 1 << 24, 128
    results, cpu_ms = measure_count(peaks, args.steps, args.warmup, variants=(2, 0, 1), big=True)
    best = min(results["uniform/variant0"], results["zipf1.1/variant0"], key=lambda r: r["gbs"])  # the slower distribution
    line = {
        "metric": "continuous_count_GBps", "value": best["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": best["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": {"workload": "count_c2", "n": n, "bins": E, "l2": "8 rotating copies of the ids (512 MB in total, larger than L2); no launch re-reads cached data",
                   "reported": "variant 0 (the default), slower of uniform / Zipf(1.1)"},
        "roofline": {"bound": "hbm", "achieved": best["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": best["gbs"] / peaks["hbm_gbs"], "traffic": n * 4, "peak_kind": peaks_kind},
        "variants": results,
        "cpu_baseline": {"value": (n * 4 + E * 4) / cpu_ms / 1e6, "unit": "GB/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": "torch.bincount of the full 2^24 ids (includes the int64 cast)"},
        "gpu_launches": _native.launch_count,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# measurement pieces shared by the main workload and the extra blocks
# ---------------------------------------------------------------------------------------------
def measure_device_steps(layer, x, dy, steps: int, warmup: int, barrier):
    """`warmup` untimed steps, then `steps` timed ones with inputs resident in HBM; returns (total ms by CUDA
    events, per-entry-point event times, kernels launched inside the timed region)."""
    from fma_b200 import _native

    for _ in range(warmup):
        layer_step(layer, x, dy)
    barrier()
    launches_before = _native.launch_count
    _native.enable_timing(True)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        layer_step(layer, x, dy)
    end.record()
    barrier()
    ms_total = start.elapsed_time(end)
    kernel_times = _native.collect_timing()
    _native.enable_timing(False)
    return ms_total, kernel_times, _native.launch_count - launches_before


# DRAM traffic of the six grouped-GEMM launches of one ep_c5 step on one GPU (bytes; dram__bytes_read.sum +
# dram__bytes_write.sum per launch from ncu captures at T = 8192, 16384 and 32768 tokens with all other
# dimensions of the workload; the traffic is linear in T - a constant for the weights plus a per-token part - and
# the fit through the two larger sizes, which predicts the smallest within 3 %, is evaluated at T = 65536).
GEMM_DRAM_TRAFFIC_EP_C5 = 75.1e9


def roofline_accounting(cfg: dict, kernel_times: dict, steps: int, ms_step: float, peaks: dict, peaks_kind: str):
    work = algorithmic_work(cfg)
    tensor_peak = peaks["bf16_tflops_sustained"] if cfg["dtype"] == "bf16" else None
    kernels = {}
    gemm_ms = 0.0
    gemm_flops = 0
    for name, (calls, ms) in sorted(kernel_times.items()):
        per_step = ms / steps
        entry = {"calls_per_step": calls / steps, "ms_per_step": per_step}
        if name in work["gemm_flops"]:
            # per-rank FLOPs: every rank processes T*k rows in expectation under a uniform router
            fl = work["gemm_flops"][name]
            entry.update(achieved=fl / per_step / 1e9, unit="TFLOP/s")
            if tensor_peak:
                entry["frac"] = entry["achieved"] / tensor_peak
            gemm_ms += per_step
            gemm_flops += fl
        elif name in work["hbm_bytes"]:
            by = work["hbm_bytes"][name]
            entry.update(achieved=by / per_step / 1e6, unit="GB/s", frac=by / per_step / 1e6 / peaks["hbm_gbs"])
        kernels[name] = entry
    roofline = None
    if gemm_ms > 0:
        achieved = gemm_flops / gemm_ms / 1e9
        traffic = GEMM_DRAM_TRAFFIC_EP_C5 if (cfg["T"], cfg["H"], cfg["E"], cfg["k"], cfg["I"]) == (65536, 4096, 128, 8, 1536) else None
        roofline = {"bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s",
                    "frac": (achieved / tensor_peak) if tensor_peak else None, "traffic": traffic,
                    "kernel": "gemm_tc2_kernel (tcgen05 cta_group::2; 6 launches per step)" if cfg["dtype"] == "bf16"
                    else "gemm_simt_kernel",
                    "peak_kind": f"{peaks_kind} sustained cuBLAS bf16", "gemm_ms_per_step": gemm_ms,
                    "gemm_share_of_step": gemm_ms / ms_step}  # fmt: skip
    return kernels, roofline


def extra_blocks(device: torch.device, peaks: dict, peaks_kind: str, steps: int = 5) -> dict:
    """Short measurements of the other single-GPU configurations, outside the timed region of the main
    workload: tokens/s and GEMM roofline fraction of the fine-grained and the Mixtral-shaped layer, GB/s of
    continuous_count at 2^24 ids.  Device-resident inputs, `steps` timed steps after 3 warm-up steps."""
    out = {}

    def barrier():
        torch.cuda.synchronize()

    for name in ("finegrained_c4", "mixtral_c3"):
        cfg = dict(WORKLOADS[name])
        layer, dtype = make_layer(cfg, 0, 1, device)
        x, dy = make_inputs(cfg, 0, device, dtype)
        x.requires_grad_(True)
        ms_total, kernel_times, _ = measure_device_steps(layer, x, dy, steps, 3, barrier)
        ms_step = ms_total / steps
        kernels, roofline = roofline_accounting(cfg, kernel_times, steps, ms_step, peaks, peaks_kind)
        out[name] = {"value": cfg["T"] / (ms_step / 1e3), "unit": "tokens/s", "ms_per_step": ms_step, "steps": steps,
                     "roofline_frac": roofline["frac"], "gemm_tflops": roofline["achieved"],
                     "gemm_frac": {k[len("fma_b200_moe_gemm_"):]: round(v["frac"], 4) for k, v in kernels.items() if "gemm" in k},
                     "hbm_frac": {k[len("fma_b200_"):]: round(v["frac"], 4) for k, v in kernels.items()
                                  if v.get("unit") == "GB/s"}}  # fmt: skip
        del layer, x, dy
        torch.cuda.empty_cache()
    results, _ = measure_count(peaks, 20, 5, variants=(0,), big=False)
    out["count_c2"] = {"unit": "GB/s", "uniform": results["uniform/variant0"], "zipf1.1": results["zipf1.1/variant0"],
                       "floor": {k.split("/")[1]: v for k, v in results.items() if k.startswith("floor/")}}
    return out


def _synthetic_counts(cfg: dict) -> list[int]:
    """Rows per expert for the GEMM comparison: R/E each under the uniform router; Zipf(1.0) loads, capped at T rows
    per expert (an expert cannot receive a token twice), for the skewed workload."""
    T, E, k = cfg["T"], cfg["E"], cfg["k"]
    R = T * k
    if cfg["router"] != "zipf":
        return [R // E] * E
    p = 1.0 / np.arange(1, E + 1)
    want = np.minimum(R * p / p.sum(), T)
    counts = np.maximum(1, np.floor(want * (R / want.sum()))).astype(np.int64)
    counts = np.minimum(counts, T)
    return [int(c) for c in counts]


def reference_gpu_block(device: torch.device, names=("ep_c5",), steps: int = 5) -> dict:
    """The six grouped GEMMs of a layer step (two forward, two dgrad, two wgrad; plain epilogues) through this
    library's entry points and through the reference project's own CUDA kernel (its CUTLASS grouped GEMM, built
    unmodified by baseline/build_reference_gemm.py, called through its stock entry point on its own unpadded
    layout), on the same GPU, same row counts, same shapes.  TFLOP/s over the token rows; ratio = ours / reference."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_gemm
    from fma_b200.modules import _kernels as K

    ok, why = reference_gemm.available()
    if ok and torch.cuda.device_count() != 1:
        ok, why = False, "the reference kernel is run by single-GPU jobs only"
    if not ok:
        return {"unavailable": why}
    try:
        reference_gemm.load()
    except Exception as e:  # missing symbol, other torch build, ...
        return {"unavailable": f"cannot load the reference kernel: {e}"[:200]}

    def timed(fn) -> float:
        for _ in range(2):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    out = {"kind": "reference CUDA kernel (CUTLASS sm100 grouped GEMM, 256x256x64 2-SM tiles), stock entry point",
           "unit": "TFLOP/s", "steps": steps}
    u32 = lambda v: torch.tensor(v, device=device, dtype=torch.uint32)  # noqa: E731
    for name in names:
        cfg = WORKLOADS[name]
        E, H, I = cfg["E"], cfg["H"], cfg["I"]
        counts = _synthetic_counts(cfg)
        rows = sum(counts)
        sel = torch.repeat_interleave(torch.arange(E), torch.tensor(counts)).view(-1, 1).to(device)
        maps = K.moe_sort(sel, E)
        M = u32(counts)
        res = {}
        tot_ours = tot_ref = 0.0
        # (label, OUT, IN) of the expert linear whose three GEMMs are timed
        for label, OUT, IN in (("c_fc", 2 * I, H), ("c_proj", H, I)):
            W = torch.randn(E, OUT, IN, device=device, dtype=torch.bfloat16) * 0.02
            Nn, Kk = u32([OUT] * E), u32([IN] * E)
            x_plain = torch.randn(rows, IN, device=device, dtype=torch.bfloat16)
            dy_plain = torch.randn(rows, OUT, device=device, dtype=torch.bfloat16)
            X = torch.randn(maps.rows_cap, IN, device=device, dtype=torch.bfloat16)
            dY = torch.randn(maps.rows_cap, OUT, device=device, dtype=torch.bfloat16)
            flops = 2.0 * rows * OUT * IN
            cases = {
                "forward": (lambda: K.gemm_forward(X, W, maps.mtile_expert),
                            lambda: reference_gemm.grouped_gemm(x_plain, W, M, Nn, Kk, (rows, OUT), False, True)),
                "dgrad": (lambda: K.gemm_dgrad(dY, W, maps.mtile_expert),
                          lambda: reference_gemm.grouped_gemm(dy_plain, W, M, Kk, Nn, (rows, IN), False, False)),
                "wgrad": (lambda: K.gemm_wgrad(dY, X, E, maps.pad_offsets),
                          lambda: reference_gemm.grouped_gemm(dy_plain, x_plain, Nn, Kk, M, (E, OUT, IN), True, False)),
            }
            for kind, (ours, ref) in cases.items():
                ms_o, ms_r = timed(ours), timed(ref)
                tot_ours += ms_o
                tot_ref += ms_r
                res[f"{label}.{kind}"] = {"ours": flops / ms_o / 1e9, "reference": flops / ms_r / 1e9,
                                          "ratio": ms_r / ms_o}
            del W, x_plain, dy_plain, X, dY
            torch.cuda.empty_cache()
        res["all_six"] = {"ours_ms": tot_ours, "reference_ms": tot_ref, "ratio": tot_ref / tot_ours}
        out[name] = res
    return out


def ep_parity_check(layer, cfg: dict, rank: int, world: int, device: torch.device, dtype, tokens: int = 1024) -> dict:
    """One small untimed step through the expert-parallel layer against a single-GPU layer that holds all
    experts (rebuilt from the same seeds) run on the tokens of all ranks: y and dx of this rank's tokens and
    the gradients of this rank's experts.  Errors are the maximum over ranks."""
    import torch.distributed as dist

    small = dict(cfg, T=tokens)
    x, dy = make_inputs(small, rank, device, dtype)
    xs = [torch.empty_like(x) for _ in range(world)]
    dys = [torch.empty_like(dy) for _ in range(world)]
    dist.all_gather(xs, x)
    dist.all_gather(dys, dy)
    full, _ = make_layer(cfg, 0, 1, device)
    x_all = torch.cat(xs).requires_grad_(True)
    y_all, _ = full(x_all)
    y_all.backward(torch.cat(dys))
    lo, hi = rank * tokens, (rank + 1) * tokens
    xr = x.clone().requires_grad_(True)
    for p in layer.parameters():
        p.grad = None
    y, _ = layer(xr)
    y.backward(dy)
    torch.cuda.synchronize()
    e0, e1 = layer.local_expert_range()

    def rel(a, b):
        return float((a.double() - b.double()).norm() / b.double().norm())

    errs = [rel(xr.grad, x_all.grad[lo:hi]), rel(layer.c_fc.weight.grad, full.c_fc.weight.grad[e0:e1]),
            rel(layer.c_proj.weight.grad, full.c_proj.weight.grad[e0:e1]), rel(y, y_all.detach()[lo:hi]),
            0.0 if torch.equal(y, y_all.detach()[lo:hi]) else 1.0]
    t = torch.tensor(errs, device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dx, dfc, dproj, ey, y_diff = t.tolist()
    for p in layer.parameters():
        p.grad = None
    del full, x_all, y_all
    torch.cuda.empty_cache()
    tol = 1e-2
    return {"tokens_per_rank": tokens, "y_bit_equal": y_diff == 0.0, "y": ey, "dx": dx, "d_w_fc": dfc, "d_w_proj": dproj,
            "tolerance": tol, "transport": layer.last_transport,
            "ok": bool(y_diff == 0.0 and max(dx, dfc, dproj) <= tol)}  # fmt: skip


# ---------------------------------------------------------------------------------------------
# main arm
# ---------------------------------------------------------------------------------------------
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="ep_c5", choices=list(WORKLOADS) + ["count_c2", "gemm_vs_reference"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="override T (for quick runs and profiler captures)")
    ap.add_argument("--ep-chunks", type=int, default=6, help="expert chunks whose exchanges overlap the GEMMs (N > 1)")
    ap.add_argument("--ep-transport", choices=["auto", "peer", "nccl"], default="auto",
                    help="row exchange of the expert-parallel layer: copy-engine pushes into peer-mapped arenas, "
                         "or NCCL all-to-all; auto = peer on 2 GPUs (if the arenas can be mapped), NCCL above (N > 1)")
    ap.add_argument("--sm-reserve", type=int, default=0, help="SMs left free for the all-to-all kernels (N > 1)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--ep-fuse-return", action="store_true",
                    help="peer transport: the down projection and the dgrad store their tiles straight into the "
                         "senders' arenas (no return copies)")
    ap.add_argument("--e2e-serial", action="store_true",
                    help="end-to-end loop with every step's copies issued inside that step; the default is a streaming "
                         "input pipeline: the host-to-device copy of step i+1 and the device-to-host copy of step i's "
                         "input gradient overlap the neighbouring step's kernels (every copy still lies inside the "
                         "timed region)")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the short extra measurements of the other single-GPU configurations (N = 1)")
    ap.add_argument("--no-ep-parity", action="store_true",
                    help="skip the small untimed parity step of the expert-parallel layer (N > 1)")
    ap.add_argument("--timeline", default="", metavar="FILE",
                    help="after the timed runs, record one more step with torch.profiler on rank 0 and write its "
                         "device timeline (start ms, duration ms, stream, kernel or copy) to FILE; never part of a "
                         "reported number")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not args.tokens else args.warmup
    peaks, peaks_kind = load_peaks()

    if args.workload == "gemm_vs_reference":
        # the six grouped GEMMs of every bf16 configuration against the reference project's own CUDA kernel
        import fma_b200  # noqa: F401

        torch.cuda.set_device(0)
        block = reference_gpu_block(torch.device("cuda:0"), ("ep_c5", "finegrained_c4", "mixtral_c3"), args.steps)
        print(json.dumps({"metric": "grouped_gemm_tflops_vs_reference_kernel", "n_gpus": 1, "reference_gpu": block}), flush=True)
        return
    if args.workload == "count_c2":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "count_c2 reports its CPU baseline inline"}))
            return
        run_count(args, peaks, peaks_kind)
        return

    cfg = dict(WORKLOADS[args.workload])
    if args.tokens:
        cfg["T"] = args.tokens
    if args.impl == "reference":
        run_reference(args, cfg, args.workload)
        return

    import fma_b200  # noqa: F401
    from fma_b200 import _native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    if world > 1 and args.workload != "ep_c5":
        raise SystemExit("only the ep_c5 workload is expert-parallel")
    device = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("TORCH_NCCL_HIGH_PRIORITY", "1")  # the exchanges must get SMs ahead of queued GEMMs
        dist.init_process_group("nccl", device_id=device)
        if args.sm_reserve > 0:
            sms = torch.cuda.get_device_properties(device).multi_processor_count
            _native.call("fma_b200_set_sm_limit", sms - args.sm_reserve)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    layer, dtype = make_layer(cfg, rank, world, device)
    if world > 1:
        layer.overlap_chunks = args.ep_chunks
        layer.transport = args.ep_transport
        layer.fuse_return = args.ep_fuse_return
    x, dy = make_inputs(cfg, rank, device, dtype)
    x.requires_grad_(True)
    T = cfg["T"]

    # ---- device-resident timing -------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    for _ in range(args.warmup):
        layer_step(layer, x, dy)
    if rank == 0:
        sampler.start()
    ms_total, kernel_times, launches = measure_device_steps(layer, x, dy, args.steps, 0, barrier)
    clocks = sampler.stop() if rank == 0 else None
    status = _native.device_status()
    if status != 0:
        raise SystemExit(f"a kernel reported device status {status:#x}")
    if world > 1:
        t = torch.tensor([ms_total], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = world * T / (ms_step / 1e3)

    # ---- end to end with host buffers -------------------------------------------------------
    e2e = None
    if not args.no_e2e:
        x_host = x.detach().cpu().pin_memory()
        dy_host = dy.detach().cpu().pin_memory()
        y_host = torch.empty_like(x_host).pin_memory()
        dx_host = torch.empty_like(x_host).pin_memory()
        copy_stream = torch.cuda.Stream(device)
        main_stream = torch.cuda.current_stream(device)

        def e2e_step():
            for p in layer.parameters():
                p.grad = None
            xd = x_host.to(device, non_blocking=True).requires_grad_(True)
            with torch.cuda.stream(copy_stream):  # dy rides along while the forward runs
                dyd = dy_host.to(device, non_blocking=True)
                dy_ready = torch.cuda.Event()
                dy_ready.record(copy_stream)
            y, _ = layer(xd)
            y_ready = torch.cuda.Event()
            y_ready.record(main_stream)
            with torch.cuda.stream(copy_stream):  # y goes back to the host while the backward runs
                copy_stream.wait_event(y_ready)
                y_host.copy_(y.detach(), non_blocking=True)
                y.record_stream(copy_stream)
            main_stream.wait_event(dy_ready)
            dyd.record_stream(main_stream)
            y.backward(dyd)
            dx_host.copy_(xd.grad, non_blocking=True)
            main_stream.wait_stream(copy_stream)  # the step ends when every copy has landed

        out_stream = torch.cuda.Stream(device)

        def e2e_loop_prefetch(n_steps: int) -> None:
            """Same copies and kernels as n_steps calls of e2e_step, as a streaming pipeline: inputs of step
            i+1 travel on copy_stream while step i computes; y and the input gradient go back on out_stream
            while the next kernels run.  The loop ends when the last copy has landed."""

            def issue_inputs():
                with torch.cuda.stream(copy_stream):
                    xd = x_host.to(device, non_blocking=True)
                    x_ready = torch.cuda.Event()
                    x_ready.record(copy_stream)
                    dyd = dy_host.to(device, non_blocking=True)  # only the backward pass needs it
                    dy_ready = torch.cuda.Event()
                    dy_ready.record(copy_stream)
                return xd, dyd, x_ready, dy_ready

            nxt = issue_inputs()
            for i in range(n_steps):
                xd, dyd, x_ready, dy_ready = nxt
                if i + 1 < n_steps:
                    nxt = issue_inputs()
                for p in layer.parameters():
                    p.grad = None
                main_stream.wait_event(x_ready)
                xd.record_stream(main_stream)
                dyd.record_stream(main_stream)
                xd.requires_grad_(True)
                y, _ = layer(xd)
                y_ready = torch.cuda.Event()
                y_ready.record(main_stream)
                with torch.cuda.stream(out_stream):
                    out_stream.wait_event(y_ready)
                    y_host.copy_(y.detach(), non_blocking=True)
                    y.record_stream(out_stream)
                main_stream.wait_event(dy_ready)
                y.backward(dyd)
                dx = xd.grad
                dx_ready = torch.cuda.Event()
                dx_ready.record(main_stream)
                with torch.cuda.stream(out_stream):
                    out_stream.wait_event(dx_ready)
                    dx_host.copy_(dx, non_blocking=True)
                    dx.record_stream(out_stream)
            main_stream.wait_stream(out_stream)

        def e2e_run(n_steps: int) -> None:
            if args.e2e_serial:
                for _ in range(n_steps):
                    e2e_step()
            else:
                e2e_loop_prefetch(n_steps)

        e2e_run(2)
        barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        e2e_run(args.steps)
        t1.record()
        barrier()
        e2e_ms = t0.elapsed_time(t1)
        if world > 1:
            t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        nbytes = x_host.numel() * x_host.element_size()
        e2e = {"value": world * T / (e2e_ms / args.steps / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * nbytes,
               "d2h_bytes_per_step": 2 * nbytes, "ms_per_step": e2e_ms / args.steps,
               "pipeline": "per-step copies" if args.e2e_serial else "inputs of step i+1 prefetched during step i"}  # fmt: skip

    timed_transport = layer.last_transport if world > 1 else None
    ep_parity = None
    if world > 1 and not args.no_ep_parity:
        ep_parity = ep_parity_check(layer, cfg, rank, world, device, dtype)

    if args.timeline:  # every rank runs the extra step; rank 0 records it
        write_timeline(args.timeline, lambda: layer_step(layer, x, dy), rank, barrier)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline accounting ----------------------------------------------------------------
    kernels, roofline = roofline_accounting(cfg, kernel_times, args.steps, ms_step, peaks, peaks_kind)

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        threads = pin_cpu_threads()
        weights = host_weights_from_layer(layer, cpu_sample(cfg)[0])
        cpu_oracle_pass(cfg, weights, seed=0, tokens=64)  # warm the BLAS threads
        secs, toks = cpu_oracle_pass(cfg, weights, seed=1)
        cpu_baseline = {"value": toks / secs, "unit": "tokens/s", "cores": threads, "kind": "port",
                        "sample": f"one forward+backward ({secs:.1f} s) of " + cpu_sample_text(cfg)}  # fmt: skip

    line = {
        "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic",
        "config": {"workload": args.workload, **{k: cfg[k] for k in ("T", "H", "E", "k", "I")},
                   "tokens_per_gpu": T, "router": cfg["router"],
                   "parallelism": f"ep{world}" if world > 1 else "single",
                   "ep_chunks": args.ep_chunks if world > 1 else None,
                   "ep_transport": timed_transport,
                   "ep_fuse_return": bool(args.ep_fuse_return) if world > 1 else None, "sm_reserve": args.sm_reserve if world > 1 else None,
                   "l2": "inputs larger than L2 (x alone is %d MB)" % (x.numel() * x.element_size() >> 20)},
        "roofline": roofline, "kernels": kernels, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks,
        "gpu_launches": launches,
    }  # fmt: skip
    if ep_parity is not None:
        line["ep_parity"] = ep_parity
    if world == 1 and args.workload == "ep_c5" and not args.tokens and not args.no_extra:
        del layer, x, dy
        torch.cuda.empty_cache()
        line["extra"] = extra_blocks(device, peaks, peaks_kind)
        line["reference_gpu"] = reference_gpu_block(device)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
