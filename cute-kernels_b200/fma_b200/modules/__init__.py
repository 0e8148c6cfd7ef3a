from .moe import Experts, MoE, grouped_gemm_experts
from .moe_ep import ExpertParallelMoE, shard_expert_state_dict, unshard_expert_state_dicts
