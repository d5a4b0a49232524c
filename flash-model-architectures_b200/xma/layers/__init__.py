from .moe import MoE, Experts
