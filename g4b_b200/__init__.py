"""g4b_b200: the attention hot path of the g4b Gemma inference engine (flash-attention
prefill, KV-cache append, split-KV decode) as hand-written CUDA for sm_100a behind the
reference's Python call signatures."""
from g4b_b200 import kernels  # noqa: F401

__all__ = ["kernels"]
