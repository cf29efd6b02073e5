from .moe import MoE, Experts, SwiGLU, SwiGLUPacked
