"""Operators of the attention hot path, named like the reference's g4b.kernels modules."""
from g4b_b200.kernels import add_kv_to_cache, advance_decode_state, fa2, rope  # noqa: F401
