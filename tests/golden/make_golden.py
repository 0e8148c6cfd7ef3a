"""Generates the golden vectors in this directory by running the REFERENCE implementation
(open-lm-engine/cute-kernels, python package `fma`, torch backend on CPU).

Run where the reference checkout is available:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/cute-kernels

The reference's MoE hard-codes the CUDA histogram even in its torch branch
(fma/modules/moe/__init__.py:215-217); the generator substitutes the reference's own torch-branch
histogram (fma/ops/continuous_count/__init__.py:35-36) for that one call and changes nothing else.
The vectors are small .npz files (bf16 tensors are stored as the float32 values they represent);
tests read them without needing the reference.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def sha16(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()[:16]


def f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().contiguous().numpy()


def build_reference_moe(fma, E, k, H, I, dtype, seed, add_bias=False):
    from fma import KernelBackend
    import fma.modules.moe as ref_moe

    ref_moe.continuous_count = lambda x, size, kernel_backend=None: fma.continuous_count(
        x, size, kernel_backend=KernelBackend.torch
    )
    act = lambda x: fma.swiglu_packed(  # noqa: E731
        x, kernel_backend_forward=KernelBackend.torch, kernel_backend_backward=KernelBackend.torch
    )
    torch.manual_seed(seed)
    moe = ref_moe.MoE(E, k, H, I, act, True, add_bias, 0.02)
    with torch.no_grad():
        moe.gate.weight.normal_(0, 0.02)
        if add_bias:  # the reference initialises biases to zero; random ones make the fixture meaningful
            moe.c_fc.bias.normal_(0, 0.5)
            moe.c_proj.bias.normal_(0, 0.5)
    return moe.to(dtype)


def run_layer(fma, T, H, E, k, I, dtype, seed, add_bias=False):
    from fma import KernelBackend

    moe = build_reference_moe(fma, E, k, H, I, dtype, seed, add_bias)
    x = torch.randn(T, H).to(dtype).requires_grad_(True)
    g = torch.randn(T, H).to(dtype)
    y, logits = moe(x, kernel_backend=KernelBackend.torch)
    y.backward(g)
    with torch.no_grad():
        _, sel = moe._get_topk(logits)
        ref_sorted_e, ref_sorted_s = sel.flatten().sort()
        st_sorted_e, st_sorted_s = sel.flatten().sort(stable=True)
        count = fma.continuous_count(ref_sorted_e, E, kernel_backend=KernelBackend.torch)
    extra = {}
    if add_bias:
        extra = {"b_fc": f32(moe.c_fc.bias), "b_proj": f32(moe.c_proj.bias), "d_b_fc": f32(moe.c_fc.bias.grad),
                 "d_b_proj": f32(moe.c_proj.bias.grad)}  # fmt: skip
    return {
        **extra,
        "x": f32(x), "g": f32(g), "w_gate": f32(moe.gate.weight), "w_fc": f32(moe.c_fc.weight),
        "w_proj": f32(moe.c_proj.weight), "y": f32(y), "router_logits": f32(logits), "dx": f32(x.grad),
        "d_w_gate": f32(moe.gate.weight.grad), "d_w_fc": f32(moe.c_fc.weight.grad),
        "d_w_proj": f32(moe.c_proj.weight.grad), "selected": sel.numpy(),
        "ref_sorted_expert_idxs": ref_sorted_e.numpy(), "ref_sorted_scattered_idxs": ref_sorted_s.numpy(),
        "stable_sorted_expert_idxs": st_sorted_e.numpy(), "stable_sorted_scattered_idxs": st_sorted_s.numpy(),
        "expert_count": count.to(torch.int64).numpy(),
    }, moe  # fmt: skip


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (the directory that holds fma/)")
    ap.add_argument("--only-bias", action="store_true",
                    help="write only the fixtures added after the first set (add_bias=True layers, the float16 layer)")
    ap.add_argument("--only-packing", action="store_true", help="write only the sequence-packing fixture")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.dont_write_bytecode = True
    import fma
    from fma import KernelBackend

    torch.set_num_threads(8)

    # ---- pack_sequence / unpack_sequence, torch backend, both padding sides -----------------------
    cu = torch.tensor([0, 3, 3, 10, 11, 18], dtype=torch.int32)  # includes an empty and a full sequence (S = 7)
    torch.manual_seed(31)
    padded = torch.randn(5, 7, 2, 4)
    packed_in = torch.randn(18, 2, 4)
    pk = {"cu_seqlens": cu.numpy(), "padded": padded.numpy(), "packed_in": packed_in.numpy()}
    for side in ("left", "right"):
        pk[f"packed_{side}"] = fma.pack_sequence(padded, cu, padding_side=side, kernel_backend_forward=KernelBackend.torch,
                                                 kernel_backend_backward=KernelBackend.torch).numpy()
        pk[f"unpacked_{side}"] = fma.unpack_sequence(packed_in, cu, (5, 7, 2, 4), padding_side=side,
                                                     kernel_backend_forward=KernelBackend.torch,
                                                     kernel_backend_backward=KernelBackend.torch).numpy()
    np.savez_compressed(HERE / "sequence_packing.npz", **pk)
    print("sequence_packing", {k: v.shape for k, v in pk.items()})
    if args.only_packing:
        return

    # ---- layer with per-expert biases (add_bias=True) ------------------------------------------
    biased = {
        "layer_f32_bias": dict(T=80, H=64, E=5, k=2, I=48, dtype=torch.float32, seed=15, add_bias=True),
        "layer_bf16_bias": dict(T=128, H=64, E=8, k=2, I=64, dtype=torch.bfloat16, seed=16, add_bias=True),
    }
    for name, cfg in biased.items():
        out, _ = run_layer(fma, **cfg)
        meta = {k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in cfg.items()}
        np.savez_compressed(HERE / f"{name}.npz", meta=json.dumps(meta), **out)
        print(name, {k: v.shape for k, v in out.items() if k in ("y", "dx", "d_b_fc")})
    # ---- layer in float16 (the reference's ops are dtype-generic: fma/include/dtypes/fp16.h) ----
    out, _ = run_layer(fma, T=96, H=64, E=8, k=2, I=32, dtype=torch.float16, seed=17)
    cfg16 = dict(T=96, H=64, E=8, k=2, I=32, dtype=str(torch.float16), seed=17)
    np.savez_compressed(HERE / "layer_f16_small.npz", meta=json.dumps(cfg16), **out)
    print("layer_f16_small", out["y"].shape)
    if args.only_bias:
        return

    # ---- layer, small shapes, every tensor stored --------------------------------------------
    small = {
        "layer_f32_small": dict(T=96, H=64, E=6, k=3, I=40, dtype=torch.float32, seed=11),
        "layer_f32_k1": dict(T=50, H=32, E=4, k=1, I=16, dtype=torch.float32, seed=12),
        "layer_bf16_small": dict(T=160, H=64, E=8, k=2, I=64, dtype=torch.bfloat16, seed=13),
        "layer_bf16_many_experts": dict(T=64, H=64, E=32, k=4, I=32, dtype=torch.bfloat16, seed=14),
    }
    for name, cfg in small.items():
        out, _ = run_layer(fma, **cfg)
        meta = {k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in cfg.items()}
        np.savez_compressed(HERE / f"{name}.npz", meta=json.dumps(meta), **out)
        print(name, {k: v.shape for k, v in out.items() if k in ("y", "dx")})

    # ---- layer, the small fp32 configuration of the benchmark spec: statistics only ------------
    out, _ = run_layer(fma, T=4096, H=1024, E=8, k=2, I=512, dtype=torch.float32, seed=0)
    stats = {"recipe": "torch.manual_seed(0); MoE(8,2,1024,512,swiglu_packed,True,False,0.02); "
                       "gate.weight.normal_(0,0.02); x=randn(4096,1024); g=randn(4096,1024)"}
    for key in ("y", "router_logits", "dx", "d_w_fc", "d_w_proj", "d_w_gate"):
        a = out[key].astype(np.float64)
        stats[key] = {"sum": float(a.sum()), "l2": float(np.linalg.norm(a)),
                      "sample": [float(v) for v in out[key].reshape(-1)[:: max(1, out[key].size // 64)][:64]]}
    stats["expert_count"] = [int(v) for v in out["expert_count"]]
    for key in ("selected", "stable_sorted_expert_idxs", "stable_sorted_scattered_idxs"):
        stats[key + "_sha16"] = hashlib.sha256(np.ascontiguousarray(out[key]).tobytes()).hexdigest()[:16]
    (HERE / "layer_f32_config1_stats.json").write_text(json.dumps(stats, indent=1))
    print("config1", stats["expert_count"], stats["y"]["sum"], stats["y"]["l2"])

    # ---- continuous_count: reference torch branch on seeded ids --------------------------------
    cc = {}
    rng = np.random.default_rng(5)
    for i, (n, size, dt) in enumerate([(0, 8, np.int32), (1, 2, np.int64), (1000, 72, np.int32), (16393, 72, np.int64),
                                       (4099, 128, np.int32), (33333, 1000, np.int64), (777, 1, np.int32)]):
        ids = rng.integers(0, size, n).astype(dt)
        ref = fma.continuous_count(torch.from_numpy(ids), size, kernel_backend=KernelBackend.torch)
        cc[f"ids_{i}"] = ids
        cc[f"size_{i}"] = np.int64(size)
        cc[f"count_{i}"] = ref.to(torch.int64).numpy()
    cc["n_cases"] = np.int64(7)
    np.savez_compressed(HERE / "continuous_count.npz", **cc)

    # ---- swiglu forward / backward --------------------------------------------------------------
    sw = {}
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        torch.manual_seed(21)
        gate = (torch.randn(37, 48) * 3).to(dtype).requires_grad_(True)
        up = torch.randn(37, 48).to(dtype).requires_grad_(True)
        dy = torch.randn(37, 48).to(dtype)
        y = fma.swiglu(gate, up, kernel_backend_forward=KernelBackend.torch, kernel_backend_backward=KernelBackend.torch)
        y.backward(dy)
        xp = torch.cat([up.detach(), gate.detach()], dim=-1)
        yp = fma.swiglu_packed(xp, kernel_backend_forward=KernelBackend.torch, kernel_backend_backward=KernelBackend.torch)
        for key, t in (("gate", gate), ("up", up), ("dy", dy), ("y", y), ("gate_grad", gate.grad), ("up_grad", up.grad),
                       ("y_packed", yp)):
            sw[f"{tag}_{key}"] = f32(t)
    np.savez_compressed(HERE / "swiglu.npz", **sw)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
