"""CPU checks of the drop-in boundary: the C-ABI library loads, exports every symbol that
include/fma_b200.h declares, argument validation works without a GPU, and the Python package keeps
the reference's names and refuses to run without CUDA (no CPU fallback)."""

import ctypes
import inspect
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "fma_b200.h"


def _declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(fma_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from fma_b200 import _native

    lib = _native.lib()
    names = _declared_symbols()
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _native.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_native.SIGNATURES) == names
    assert lib.fma_b200_abi_version() == 3


def test_status_strings_and_bad_arguments_without_gpu():
    from fma_b200 import _native

    lib = _native.lib()
    assert lib.fma_b200_status_string(0) == b"ok"
    assert b"unknown" in lib.fma_b200_status_string(999)
    null = ctypes.c_void_p(None)
    # argument checks run before any CUDA call, so they work on a machine without a GPU
    assert lib.fma_b200_continuous_count(null, 4, 10, 0, null, null, 0, null) == 1
    assert b"NULL" in lib.fma_b200_last_error() or b"size" in lib.fma_b200_last_error()
    assert lib.fma_b200_continuous_count(null, 2, 0, 8, null, null, 0, null) == 1
    assert lib.fma_b200_router_topk_softmax(null, 0, 4, 8, 9, null, null, null) == 1  # k > E
    assert lib.fma_b200_moe_gemm_forward(null, null, null, 7, 128, 2, 8, 8, null, 128, null) == 2  # dtype
    assert lib.fma_b200_moe_gemm_forward(null, null, null, 1, 100, 2, 8, 8, null, 128, null) == 1  # rows_cap % 128
    assert lib.fma_b200_moe_gemm_forward_swiglu(null, null, null, null, 0, 128, 2, 8, 8, null, 128, null) == 2  # f32
    with pytest.raises(RuntimeError, match="bad argument"):
        _native.call("fma_b200_swiglu_forward", null, 8, null, 8, null, 8, 1, 4, 12, null)  # cols % 8
    assert lib.fma_b200_moe_rows_cap(1000, 8, 128) == 2048
    assert lib.fma_b200_moe_rows_cap(1000, 8, 256) == 3072
    assert lib.fma_b200_moe_rows_cap(0, 1, 128) == 128
    assert lib.fma_b200_continuous_count_workspace_bytes(128) == 128 + 8 * 128 * 4
    # expert bias and the peer-memory transport
    assert lib.fma_b200_moe_bias_add(null, null, 7, 128, 64, null, null, null) == 2  # dtype
    assert lib.fma_b200_moe_bias_add(null, null, 1, 128, 12, null, null, null) == 1  # width not 16-byte multiple
    assert lib.fma_b200_moe_bias_add(null, null, 1, 0, 64, null, null, null) == 0  # nothing to do
    assert lib.fma_b200_moe_bias_grad(null, 1, 0, 64, null, null, null) == 1  # E < 1
    assert lib.fma_b200_moe_gemm_forward_peer(null, null, null, 0, 256, 2, 64, 64, null, 256, null) == 2  # f32
    assert lib.fma_b200_moe_gemm_forward_peer(null, null, null, 1, 256, 2, 64, 64, null, 128, null) == 2  # row_align
    assert lib.fma_b200_moe_gemm_dgrad_peer(null, null, null, 1, 256, 2, 64, 64, null, 256, null) == 1  # NULL pointers
    assert lib.fma_b200_moe_gemm_dgrad_peer(null, null, null, 1, 0, 2, 64, 64, null, 256, null) == 0  # no rows
    assert lib.fma_b200_peer_buffer_create(0, null, null) == 1
    assert lib.fma_b200_peer_buffer_open(null, null) == 1
    assert lib.fma_b200_peer_copy(0, null, null, null, null) == 0
    assert lib.fma_b200_peer_copy(-1, null, null, null, null) == 1
    one = (ctypes.c_uint64 * 1)(0)
    assert lib.fma_b200_peer_copy(1, one, one, (ctypes.c_int64 * 1)(16), null) == 1  # NULL address
    assert lib.fma_b200_peer_signal(65, one, 1, null) == 1  # more than 64 flags
    assert lib.fma_b200_peer_signal(1, one, 1, null) == 1  # NULL flag address
    assert lib.fma_b200_peer_wait(null, 1, 1, 1000, null) == 1
    assert lib.fma_b200_peer_wait(one, 1, 1, 0, null) == 1  # no unbounded waits
    assert lib.fma_b200_peer_wait(one, 1, 1, 600000, null) == 1


def test_python_surface_matches_reference_names():
    import fma_b200
    from fma_b200 import KernelBackend, MoE

    assert [b.value for b in KernelBackend] == ["cuda", "torch", "triton"]
    sig = inspect.signature(MoE.__init__)
    assert list(sig.parameters)[1:] == ["num_experts", "num_experts_per_tok", "hidden_size", "intermediate_size",
                                        "activation_function", "is_glu", "add_bias", "std"]
    assert list(inspect.signature(MoE.forward).parameters) == ["self", "hidden_states", "kernel_backend"]
    assert list(inspect.signature(fma_b200.continuous_count).parameters)[:3] == ["x", "size", "kernel_backend"]
    gg = list(inspect.signature(fma_b200.grouped_gemm).parameters)
    assert gg == ["A", "B", "C", "M_array", "N_array", "K_array", "output_shape", "alpha", "beta", "is_A_transposed",
                  "is_B_transposed", "benchmark"]
    assert list(inspect.signature(fma_b200.swiglu).parameters) == ["gate", "up", "kernel_backend_forward",
                                                                   "kernel_backend_backward"]
    moe = MoE(8, 2, 64, 32, fma_b200.swiglu_packed, True, False, 0.02)
    assert list(moe.state_dict()) == ["gate.weight", "c_fc.weight", "c_fc.N_array", "c_fc.K_array", "c_proj.weight",
                                      "c_proj.N_array", "c_proj.K_array"]
    assert moe.c_fc.weight.shape == (8, 64, 64) and moe.c_proj.weight.shape == (8, 64, 32)
    assert moe.c_fc.N_array.dtype == torch.uint32 and moe.c_fc.N_array.tolist() == [64] * 8
    assert moe.c_proj.K_array.tolist() == [32] * 8
    # round trip through a state dict, strict
    other = MoE(8, 2, 64, 32, fma_b200.swiglu_packed, True, False, 0.02)
    other.load_state_dict(moe.state_dict(), strict=True)
    assert torch.equal(other.c_fc.weight, moe.c_fc.weight)


def test_no_cpu_fallback():
    import fma_b200

    moe = fma_b200.MoE(4, 2, 32, 16, fma_b200.swiglu_packed, True, False, 0.02)
    with pytest.raises(RuntimeError, match="CUDA"):
        moe(torch.randn(3, 32))
    with pytest.raises(RuntimeError, match="CUDA"):
        fma_b200.continuous_count(torch.zeros(5, dtype=torch.int32), 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        fma_b200.swiglu(torch.randn(2, 8), torch.randn(2, 8))
    with pytest.raises(ValueError):
        moe(torch.randn(3, 32), kernel_backend="cuda")


def test_product_never_imports_the_oracle():
    pkg = ROOT / "cute-kernels_b200"
    for path in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.cuh")):
        text = path.read_text()
        assert "oracle" not in text.lower(), f"{path} mentions the oracle"
        assert "_work/" not in text, f"{path} refers to working files"
