from .moe import Experts, MoE
from .moe_ep import ExpertParallelMoE, shard_expert_state_dict, unshard_expert_state_dicts
