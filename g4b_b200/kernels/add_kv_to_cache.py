"""add_kv_to_cache: the reference's call signature (g4b/kernels/add_kv_to_cache.py:162-170)
over the CUDA library, plus the paged destination."""
from __future__ import annotations

import ctypes

from g4b_b200 import _cabi


def add_kv_to_cache(
    x,
    cache,
    cache_offsets,
    rmsnorm_eps: float,
    x_rsos=None,
    user_phase=None,
    phase: int = 0,
    *,
    block_tables=None,
    page_size: int = 16,
    stream=None,
):
    """``cache[b, g, (cache_offsets[b] + t) % T, :] = x[b, g, t, :]`` cast to the cache dtype,
    times ``rsqrt(x_rsos[b,g,t] / D + rmsnorm_eps)`` when ``x_rsos`` is given
    (add_kv_to_cache.py:148-158).  With ``block_tables [B,max_pages]`` the cache is a page pool
    ``[num_pages,G,page_size,D]`` and token ``p = cache_offsets[b] + t`` goes to page
    ``block_tables[b, p // page_size]``, row ``p % page_size``.  Slots whose ``user_phase``
    differs from ``phase`` are skipped.  Returns None."""
    assert isinstance(phase, int)
    a = _cabi.G4bAppendArgs()
    a.x = _cabi.as_tensor(x)
    a.cache = _cabi.as_tensor(cache)
    a.cache_offsets = _cabi.as_tensor(cache_offsets)
    a.x_rsos = _cabi.as_tensor(x_rsos)
    a.user_phase = _cabi.as_tensor(user_phase)
    a.block_tables = _cabi.as_tensor(block_tables)
    a.rmsnorm_eps = float(rmsnorm_eps)
    a.phase = int(phase)
    a.page_size = int(page_size)
    _cabi.check(_cabi.load().g4b_kv_append(ctypes.byref(a), ctypes.c_void_p(_cabi.current_stream(stream))))
    return None


def add_kv_to_cache_fp8(x, cache, scales, cache_offsets, rmsnorm_eps, x_rsos=None, user_phase=None, phase=0, *,
                        block_tables, page_size: int = 16, headroom: float = 2.0, stream=None):
    """``add_kv_to_cache`` into an 8-bit (e4m3) page pool ``[num_pages,G,page,D]`` with one f32 scale
    per (page, kv head) in ``scales [num_pages,G]`` (``g4b_kv_append_fp8``).  A page's scale is
    fixed by its first row: ``max|row| x headroom / 448``; every row of the page is stored as
    round-to-nearest, saturating e4m3 of ``row / scale``.  No counterpart in the reference."""
    import ctypes

    a = _cabi.G4bFp8AppendArgs()
    a.x = _cabi.as_tensor(x)
    a.cache = _cabi.as_tensor(cache)
    a.scales = _cabi.as_tensor(scales)
    a.cache_offsets = _cabi.as_tensor(cache_offsets)
    a.x_rsos = _cabi.as_tensor(x_rsos)
    a.user_phase = _cabi.as_tensor(user_phase)
    a.block_tables = _cabi.as_tensor(block_tables)
    a.rmsnorm_eps, a.headroom = float(rmsnorm_eps), float(headroom)
    a.phase, a.page_size = int(phase), int(page_size)
    _cabi.check(_cabi.load().g4b_kv_append_fp8(ctypes.byref(a), ctypes.c_void_p(_cabi.current_stream(stream))))
    return None


def dequantise_fp8_pool(cache, scales, out, *, block_tables=None, time_dim_sizes=None, user_phase=None, phase=0,
                        page_size: int = 16, stream=None):
    """An 8-bit (e4m3) page pool into a 16-bit pool of the same geometry, page for page
    (``g4b_kv_dequant_fp8``): ``out[p] = round(e4m3(cache[p]) x scales[p])``, so the same block
    tables address both and a prefill chunk (``fa2.flash_attention`` with Tq > 1) can attend to a
    context that lives in 8 bits.  With ``block_tables`` and ``time_dim_sizes`` only the pages that
    hold the slots' first ``time_dim_sizes[b]`` tokens are converted (of the slots in ``phase``,
    when ``user_phase`` is given).  No counterpart in the reference."""
    import ctypes

    a = _cabi.G4bFp8DequantArgs()
    a.cache = _cabi.as_tensor(cache)
    a.scales = _cabi.as_tensor(scales)
    a.out = _cabi.as_tensor(out)
    a.block_tables = _cabi.as_tensor(block_tables)
    a.time_dim_sizes = _cabi.as_tensor(time_dim_sizes)
    a.user_phase = _cabi.as_tensor(user_phase)
    a.phase, a.page_size = int(phase), int(page_size)
    _cabi.check(_cabi.load().g4b_kv_dequant_fp8(ctypes.byref(a), ctypes.c_void_p(_cabi.current_stream(stream))))
    return None
