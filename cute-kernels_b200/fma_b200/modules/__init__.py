from .moe import Experts, MoE
