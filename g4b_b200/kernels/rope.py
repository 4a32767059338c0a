"""apply_rope with the reference's call signature (g4b/kernels/rope.py:214-247), and the fused
form that also normalises V and appends K and V to the cache in the same launch."""
from __future__ import annotations

import ctypes

from g4b_b200 import _cabi


def _launch(a, stream):
    _cabi.check(_cabi.load().g4b_rope_norm_append(ctypes.byref(a), ctypes.c_void_p(_cabi.current_stream(stream))))


def apply_rope(
    q,
    k,
    rope_freqs,
    time_dim_offsets,
    q_rsos,
    k_rsos,
    q_rmsnorm_w,
    k_rmsnorm_w,
    rmsnorm_eps: float,
    *,
    stream=None,
):
    """In place on ``q [B,H,t,D]`` and ``k [B,G,t,D]``: each row is scaled by
    ``rsqrt(rsos / D + eps) * w`` and its element pairs ``(i, i + D/2)`` are rotated by
    ``theta = (time_dim_offsets[b] + t) * rope_freqs[i]`` (rope.py:22-39,166-173).  Returns None."""
    a = _cabi.G4bRopeAppendArgs()
    a.q = _cabi.as_tensor(q)
    a.k = _cabi.as_tensor(k)
    a.rope_freqs = _cabi.as_tensor(rope_freqs)
    a.cache_offsets = _cabi.as_tensor(time_dim_offsets)
    a.q_rsos = _cabi.as_tensor(q_rsos)
    a.k_rsos = _cabi.as_tensor(k_rsos)
    a.q_norm_w = _cabi.as_tensor(q_rmsnorm_w)
    a.k_norm_w = _cabi.as_tensor(k_rmsnorm_w)
    a.rmsnorm_eps = float(rmsnorm_eps)
    a.norm_qk = 1
    _launch(a, stream)
    return None


def rope_norm_append(
    q,
    k,
    v,
    rope_freqs,
    cache_offsets,
    k_cache,
    v_cache,
    rmsnorm_eps: float,
    *,
    q_out=None,
    k_out=None,
    q_rsos=None,
    k_rsos=None,
    v_rsos=None,
    q_rmsnorm_w=None,
    k_rmsnorm_w=None,
    norm_qk: bool = True,
    norm_v: bool = True,
    user_phase=None,
    phase: int = 0,
    block_tables=None,
    page_size: int = 16,
    stream=None,
):
    """One launch for ``apply_rope(q, k, ...)``, ``add_kv_to_cache(k, k_cache, ...)`` and
    ``add_kv_to_cache(v, v_cache, ..., v_rsos)`` (the sequence at g4b/models/gemma4e.py:564-592).

    The rotated q goes to ``q_out`` (any float dtype) or back into ``q``; the rotated k goes to
    ``k_cache`` for slots in ``phase`` (and to ``k_out`` if given); v, scaled by
    ``rsqrt(rsos / D + eps)``, goes to ``v_cache``.  Sums of squares that are not passed are
    computed from the rows.  ``block_tables`` makes the caches page pools."""
    assert isinstance(phase, int)
    a = _cabi.G4bRopeAppendArgs()
    a.q = _cabi.as_tensor(q)
    a.k = _cabi.as_tensor(k)
    a.v = _cabi.as_tensor(v)
    a.q_out = _cabi.as_tensor(q_out)
    a.k_out = _cabi.as_tensor(k_out)
    a.rope_freqs = _cabi.as_tensor(rope_freqs)
    a.cache_offsets = _cabi.as_tensor(cache_offsets)
    a.q_rsos = _cabi.as_tensor(q_rsos)
    a.k_rsos = _cabi.as_tensor(k_rsos)
    a.v_rsos = _cabi.as_tensor(v_rsos)
    a.q_norm_w = _cabi.as_tensor(q_rmsnorm_w)
    a.k_norm_w = _cabi.as_tensor(k_rmsnorm_w)
    a.k_cache = _cabi.as_tensor(k_cache)
    a.v_cache = _cabi.as_tensor(v_cache)
    a.user_phase = _cabi.as_tensor(user_phase)
    a.block_tables = _cabi.as_tensor(block_tables)
    a.rmsnorm_eps = float(rmsnorm_eps)
    a.phase = int(phase)
    a.page_size = int(page_size)
    a.norm_qk = 1 if norm_qk else 0
    a.norm_v = 1 if norm_v else 0
    _launch(a, stream)
    return None
