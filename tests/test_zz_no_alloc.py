"""The allocation-free decode entry point (g4b_attn_decode_static_scratch), called through
the C ABI, against the ordinary entry point that takes caller-provided partial buffers.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  It passes on its own in a fresh process and after the other tests."""
import pytest
import torch

from g4b_b200.kernels import fa2
from helpers import assert_close, make_paged_case, make_ring_case


def _reference_call(case, cuda, splits, layout):
    q = case["q"].to(cuda)
    B, H, Tq, D = q.shape
    o = torch.zeros(B, H, Tq, D, dtype=q.dtype, device=cuda)
    po = torch.empty(splits, B, H, Tq, D, device=cuda)
    pl = torch.empty(splits, B, H, Tq, device=cuda)
    pm = torch.empty(splits, B, H, Tq, device=cuda)
    if layout == "paged":
        fa2.flash_attention(q, case["k_pool"].to(cuda), case["v_pool"].to(cuda), o, case["time"].to(cuda), None,
                            case["max_len"], fa2.PHASE_DECODE, po, pl, pm, scale=1 / 16,
                            block_tables=case["block_tables"].to(cuda), page_size=16, num_kv_splits=splits)
    else:
        fa2.flash_attention(q, case["k"].to(cuda), case["v"].to(cuda), o, case["time"].to(cuda), None,
                            case["ctx_window"], fa2.PHASE_DECODE, po, pl, pm, scale=1 / 16, num_kv_splits=splits)
    return o


def _static_call(case, cuda, splits, layout):
    q = case["q"].to(cuda)
    o = torch.zeros_like(q)
    if layout == "paged":
        fa2.decode_attention_static_scratch(q, case["k_pool"].to(cuda), case["v_pool"].to(cuda), o,
                                            case["time"].to(cuda), None, case["max_len"], fa2.PHASE_DECODE,
                                            scale=1 / 16, block_tables=case["block_tables"].to(cuda), page_size=16,
                                            num_kv_splits=splits)
    else:
        fa2.decode_attention_static_scratch(q, case["k"].to(cuda), case["v"].to(cuda), o, case["time"].to(cuda), None,
                                            case["ctx_window"], fa2.PHASE_DECODE, scale=1 / 16, num_kv_splits=splits)
    return o


@pytest.mark.gpu
def test_static_scratch_decode_matches_caller_buffers_twice(cuda):
    """Two calls in a row on different inputs and split counts: the second must not see
    anything the first left in the shared array."""
    first = make_paged_case(71, lens=[3000, 17, 555, 4096], H=8, G=2, dtype=torch.float16)
    second = make_ring_case(72, B=3, H=8, G=2, Tq=1, T=2048, dtype=torch.bfloat16)
    for case, splits, layout in ((first, 16, "paged"), (second, 5, "ring")):
        want = _reference_call(case, cuda, splits, layout)
        got = _static_call(case, cuda, splits, layout)
        assert_close(got, want.float(), f"static scratch, {layout}, {splits} splits")
    # and once more on the first inputs, now that the array holds the second call's partials
    assert_close(_static_call(first, cuda, 16, "paged"), _reference_call(first, cuda, 16, "paged").float(),
                 "static scratch, repeat")


def test_static_scratch_rejects_sizes_beyond_its_maximum():
    """Beyond 16 splits or 8192 workspace rows the call fails with a clear message before it
    touches the GPU."""
    B, H, G, D, T = 80, 8, 2, 256, 64          # 16 splits x 80 x 8 = 10240 rows > 8192
    q = torch.zeros(B, H, 1, D, dtype=torch.float16)
    k = torch.zeros(B, G, T, D, dtype=torch.float16)
    time = torch.full((B,), T, dtype=torch.int32)
    with pytest.raises(ValueError, match="static decode workspace too small.*8192 rows"):
        fa2.decode_attention_static_scratch(q, k, k, torch.zeros_like(q), time, None, T, 2, num_kv_splits=16, stream=0)
    with pytest.raises(ValueError, match="maximum is 16 splits"):
        fa2.decode_attention_static_scratch(q[:1], k[:1], k[:1], torch.zeros_like(q[:1]), time[:1], None, T, 2,
                                            num_kv_splits=17, stream=0)
    with pytest.raises(ValueError, match="takes no partial buffers"):
        import ctypes
        from g4b_b200 import _cabi
        a = fa2._attn_args(q[:1], k[:1], k[:1], torch.zeros_like(q[:1]), time[:1], None, T, 2,
                           torch.zeros(2, 1, H, 1, D), torch.zeros(2, 1, H, 1), torch.zeros(2, 1, H, 1),
                           3, 1.0, None, None, 16, 2)
        _cabi.check(_cabi.load().g4b_attn_decode_static_scratch(ctypes.byref(a), ctypes.c_void_p(0)))
