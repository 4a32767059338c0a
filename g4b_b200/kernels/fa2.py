"""flash_attention: the reference's call signature (g4b/kernels/fa2.py:634-652) over the
CUDA library.

Drop-in defaults reproduce the reference kernel: no softmax scale (fa2.py:89), the window
shared by a chunk's queries (fa2.py:52-67), ring-buffer caches.  Keyword-only extras select
what the reference does not have: ``scale``, a per-query ``sliding_window`` (the semantics of
scripts/reference_impl.py:437-443), paged caches through ``block_tables`` and a forced split
count.
"""
from __future__ import annotations

import ctypes

from g4b_b200 import _cabi

# g4b/kernels/fa2.py:14-16
STAGE_FULL = 1
STAGE_ON_BAND = 2
STAGE_CAUSAL = STAGE_FULL | STAGE_ON_BAND
# g4b/kernels/fa2.py:29-31
PHASE_UNALLOCATED = 0
PHASE_PREFILL = 1
PHASE_DECODE = 2


def select_kv_splits(ctx_window_size: int, max_kv_splits: int, phase: int, tq: int) -> int:
    """Split count the library picks when none is forced (policy of fa2.py:186-225)."""
    return int(_cabi.load().g4b_select_kv_splits(int(ctx_window_size), int(max_kv_splits), int(phase), int(tq)))


def _attn_args(q, k_cache, v_cache, o, time_dim_sizes, user_phase, ctx_window_size, phase,
               partial_o, partial_l, partial_m, stage, scale, sliding_window, block_tables,
               page_size, num_kv_splits) -> _cabi.G4bAttnArgs:
    a = _cabi.G4bAttnArgs()
    a.q = _cabi.as_tensor(q)
    a.k_cache = _cabi.as_tensor(k_cache)
    a.v_cache = _cabi.as_tensor(v_cache)
    a.o = _cabi.as_tensor(o)
    a.time_dim_sizes = _cabi.as_tensor(time_dim_sizes)
    a.user_phase = _cabi.as_tensor(user_phase)
    a.partial_o = _cabi.as_tensor(partial_o)
    a.partial_l = _cabi.as_tensor(partial_l)
    a.partial_m = _cabi.as_tensor(partial_m)
    a.block_tables = _cabi.as_tensor(block_tables)
    a.ctx_window_size = int(ctx_window_size)
    a.phase = int(phase)
    a.stage = int(stage)
    a.page_size = int(page_size)
    a.sliding_window = int(sliding_window or 0)
    a.num_kv_splits = int(num_kv_splits or 0)
    a.scale = float(scale)
    return a


def flash_attention(
    q,
    k_cache,
    v_cache,
    o,
    time_dim_sizes,
    user_phase,
    ctx_window_size: int,
    phase: int,
    partial_o=None,
    partial_l=None,
    partial_m=None,
    *,
    use_grouped_query_tile: bool = True,
    warp_specialize: bool = False,
    is_hopper: bool = False,
    use_fp32_dot: bool = False,
    stage: int = STAGE_CAUSAL,
    scale: float = 1.0,
    sliding_window: int | None = None,
    block_tables=None,
    page_size: int = 16,
    num_kv_splits: int | None = None,
    stream=None,
):
    """Attention of ``q [B,H,Tq,D]`` over a KV cache into ``o``; returns None.

    Ring mode (reference): ``k_cache, v_cache [B,G,T,D]``; slot b exposes its last
    ``min(time_dim_sizes[b], ctx_window_size)`` keys, stored at rows
    ``(ring_start + j) % T`` (fa2.py:52-55,75).  Paged mode: pass ``block_tables [B,max_pages]``
    and pools ``[num_pages,G,page_size,D]``.  Slots whose ``user_phase`` differs from ``phase``
    are left untouched (fa2.py:333-335).  With a complete ``partial_*`` triple a Tq == 1 call
    may split the key range and merge the parts (fa2.py:702-714).

    ``use_grouped_query_tile``, ``warp_specialize``, ``is_hopper`` and ``use_fp32_dot`` tune the
    reference's Triton kernel; they are accepted and have no effect here (query heads of a kv
    head always share its K/V traffic, accumulation is always f32).
    """
    assert isinstance(phase, int)
    if (partial_o is None) != (partial_l is None) or (partial_o is None) != (partial_m is None):
        raise ValueError("partial_o, partial_l, and partial_m must be provided together")
    a = _attn_args(q, k_cache, v_cache, o, time_dim_sizes, user_phase, ctx_window_size, phase,
                   partial_o, partial_l, partial_m, stage, scale, sliding_window, block_tables,
                   page_size, num_kv_splits)
    _cabi.check(_cabi.load().g4b_flash_attention(ctypes.byref(a), ctypes.c_void_p(_cabi.current_stream(stream))))
    return None


def attention_decode_partials(q, k_cache, v_cache, o, time_dim_sizes, user_phase, ctx_window_size,
                              phase, partial_o, partial_l, partial_m, num_kv_splits, *, scale=1.0,
                              sliding_window=None, block_tables=None, page_size=16,
                              stage=STAGE_CAUSAL, stream=None):
    """Runs only the Tq == 1 kernel: with ``num_kv_splits > 1`` it fills the first
    ``num_kv_splits`` entries of the partial buffers (un-normalised acc, l, m in log2 units,
    fa2.py:438-472) and does not merge them -- the caller merges, e.g. after gathering the
    partials of other GPUs."""
    a = _attn_args(q, k_cache, v_cache, o, time_dim_sizes, user_phase, ctx_window_size, phase,
                   partial_o, partial_l, partial_m, stage, scale, sliding_window, block_tables,
                   page_size, num_kv_splits)
    _cabi.check(_cabi.load().g4b_attn_decode(ctypes.byref(a), ctypes.c_void_p(_cabi.current_stream(stream))))


def decode_step(q, k_cache, v_cache, o, time_dim_sizes, user_phase, ctx_window_size, phase, partial_o, partial_l,
                partial_m, *, k_new=None, v_new=None, exchange=None, num_kv_splits=None, scale=1.0,
                sliding_window=None, block_tables=None, page_size=16, stage=STAGE_CAUSAL, stream=None):
    """The decode step of one attention layer (``g4b_decode_step``): what the reference issues as
    two add_kv_to_cache launches, the attention launch and the split-KV reduce launch
    (g4b/models/gemma4e.py:575-607, fa2.py:702-714) as two launches -- attention with the append
    inside it, then the merge, scheduled while the first drains -- or, with ``exchange``, as one.

    ``q [B,H,1,D]``; ``partial_*`` (f32) are the split workspace.  ``k_new, v_new [B,G,1,D]``
    (cache dtype), if given, are written to the cache at position ``time_dim_sizes[b] - 1`` of
    every slot in phase and attended to.  ``exchange`` (a ``g4b_b200.dist.PartialExchange``):
    this rank holds only its share of one sequence's keys; the local splits are merged, the
    merged partials of all ranks are exchanged through peer memory and merged again, all in the
    attention launch.  That form counts its CTAs in two words inside the library, one pair per
    GPU: calls with ``exchange`` that overlap on one GPU (two streams) would share them -- keep
    them on one stream or order them."""
    if (k_new is None) != (v_new is None):
        raise ValueError("k_new and v_new must be given together")
    s = _cabi.G4bDecodeStepArgs()
    s.attn = _attn_args(q, k_cache, v_cache, o, time_dim_sizes, user_phase, ctx_window_size, phase,
                        partial_o, partial_l, partial_m, stage, scale, sliding_window, block_tables,
                        page_size, num_kv_splits)
    s.k_new = _cabi.as_tensor(k_new)
    s.v_new = _cabi.as_tensor(v_new)
    s.world, s.rank = 0, 0
    if exchange is not None:
        for r in range(exchange.world):
            s.xbuf[r] = exchange.xbuf_ptrs[r]
        s.state = exchange.state.data_ptr()
        s.xbuf_bytes = exchange.xbuf_bytes
        s.world, s.rank = exchange.world, exchange.rank
    _cabi.check(_cabi.load().g4b_decode_step(ctypes.byref(s), ctypes.c_void_p(_cabi.current_stream(stream))))


def flash_attention_fp8(q, k_pool, v_pool, k_scales, v_scales, o, time_dim_sizes, user_phase, ctx_window_size,
                        phase, partial_o=None, partial_l=None, partial_m=None, *, block_tables, page_size=16,
                        scale=1.0, sliding_window=None, num_kv_splits=None, stage=STAGE_CAUSAL, stream=None):
    """Tq == 1 attention over 8-bit (e4m3) page pools ``[num_pages,G,page,D]`` with one f32 scale per
    (page, kv head), ``k_scales / v_scales [num_pages,G]``: the attention of ``flash_attention`` on the
    values ``e4m3(byte) x scale`` (``g4b_flash_attention_fp8``).  The reference has no 8-bit
    cache; pools are filled by ``add_kv_to_cache_fp8``."""
    if (partial_o is None) != (partial_l is None) or (partial_o is None) != (partial_m is None):
        raise ValueError("partial_o, partial_l, and partial_m must be provided together")
    a = _attn_args(q, k_pool, v_pool, o, time_dim_sizes, user_phase, ctx_window_size, phase,
                   partial_o, partial_l, partial_m, stage, scale, sliding_window, block_tables,
                   page_size, num_kv_splits)
    ks, vs = _cabi.as_tensor(k_scales), _cabi.as_tensor(v_scales)
    _cabi.check(_cabi.load().g4b_flash_attention_fp8(ctypes.byref(a), ctypes.byref(ks), ctypes.byref(vs),
                                                     ctypes.c_void_p(_cabi.current_stream(stream))))


def combine_partials(partial_o, partial_l, partial_m, o, num_splits, *, user_phase=None, phase=0, stream=None):
    """Log-sum-exp merge of ``num_splits`` partials into ``o`` (fa2.py:546-631)."""
    c = _cabi.G4bCombineArgs()
    c.partial_o = _cabi.as_tensor(partial_o)
    c.partial_l = _cabi.as_tensor(partial_l)
    c.partial_m = _cabi.as_tensor(partial_m)
    c.o = _cabi.as_tensor(o)
    c.user_phase = _cabi.as_tensor(user_phase)
    c.num_splits = int(num_splits)
    c.phase = int(phase)
    _cabi.check(_cabi.load().g4b_attn_combine(ctypes.byref(c), ctypes.c_void_p(_cabi.current_stream(stream))))


def decode_attention_static_scratch(q, k_cache, v_cache, o, time_dim_sizes, user_phase, ctx_window_size, phase, *,
                                    scale=1.0, sliding_window=None, block_tables=None, page_size=16,
                                    num_kv_splits=None, stage=STAGE_CAUSAL, stream=None):
    """Tq == 1 attention with split-KV for callers that may not allocate device memory (a
    serving loop with a memory budget fixed at load, a plugin inside an engine that owns every
    buffer): the split workspace is a fixed 8 MiB array inside the library instead of
    caller-provided partial buffers.  Limits: head dim 256, at most 16 splits and
    splits * B * H <= 8192, else ValueError.  Calls share that array, so run them on one stream
    (or otherwise ordered); the first call on a device should precede any stream capture."""
    a = _attn_args(q, k_cache, v_cache, o, time_dim_sizes, user_phase, ctx_window_size, phase,
                   None, None, None, stage, scale, sliding_window, block_tables, page_size, num_kv_splits)
    _cabi.check(_cabi.load().g4b_attn_decode_static_scratch(ctypes.byref(a),
                                                            ctypes.c_void_p(_cabi.current_stream(stream))))
