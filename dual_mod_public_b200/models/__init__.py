from .attention import DualModAttention
from .layers import LoRAGate, LoRALinear, RMSNorm, SwiGLU
from .lm import Block, DualModLM
from .rope import apply_rope, build_rope_cache
from .scan import sequential_scan

__all__ = ["DualModAttention", "DualModLM", "Block", "RMSNorm", "SwiGLU", "LoRAGate",
           "LoRALinear", "apply_rope", "build_rope_cache", "sequential_scan"]
