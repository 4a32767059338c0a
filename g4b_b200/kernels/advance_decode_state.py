"""advance_decode_state: the reference's call signature
(g4b/kernels/advance_decode_state.py:66-72) over the CUDA library."""
from __future__ import annotations

import ctypes

from g4b_b200 import _cabi


def advance_decode_state(input_token_ids, out_token_ids, cache_offsets, time_dim_sizes, user_phase, *, stream=None):
    """For every slot in the decode phase: feed the sampled token back
    (``input_token_ids[0,b] = out_token_ids[b,0]``) and advance ``cache_offsets[b]`` and
    ``time_dim_sizes[b]`` by one (advance_decode_state.py:52-63).  Returns None."""
    a = _cabi.G4bAdvanceArgs()
    a.input_token_ids = _cabi.as_tensor(input_token_ids)
    a.out_token_ids = _cabi.as_tensor(out_token_ids)
    a.cache_offsets = _cabi.as_tensor(cache_offsets)
    a.time_dim_sizes = _cabi.as_tensor(time_dim_sizes)
    a.user_phase = _cabi.as_tensor(user_phase)
    _cabi.check(_cabi.load().g4b_advance_decode_state(ctypes.byref(a), ctypes.c_void_p(_cabi.current_stream(stream))))
    return None
