"""B200-native (sm_100a) implementation of the MoE-layer hot path of open-lm-engine/cute-kernels.

Drop-in names: `MoE`, `Experts`, `continuous_count`, `grouped_gemm`, `swiglu`, `swiglu_packed`,
`pack_sequence`, `unpack_sequence`, `KernelBackend`.  All compute runs in hand-written CUDA kernels loaded from libfma_b200.so through a
C ABI (see include/fma_b200.h); there is no Triton, eager-PyTorch or CPU fallback.
"""

from . import _native
from .kernel_backend import KernelBackend
from .modules import Experts, ExpertParallelMoE, MoE, shard_expert_state_dict, unshard_expert_state_dicts
from .ops import continuous_count, grouped_gemm, pack_sequence, swiglu, swiglu_packed, unpack_sequence
from .utils import ceil_divide, ensure_contiguous, set_seed

__all__ = [
    "KernelBackend",
    "MoE",
    "Experts",
    "ExpertParallelMoE",
    "shard_expert_state_dict",
    "unshard_expert_state_dicts",
    "continuous_count",
    "grouped_gemm",
    "swiglu",
    "swiglu_packed",
    "pack_sequence",
    "unpack_sequence",
    "ensure_contiguous",
    "set_seed",
    "ceil_divide",
]
