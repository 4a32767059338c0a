"""The allocation-free decode entry point (g4b_attn_decode_static_scratch), called through
the C ABI, against the ordinary entry point that takes caller-provided partial buffers and
against the CPU oracle; the free device memory must be the same before and after a call.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  It passes on its own in a fresh process and after the other tests."""
import pytest
import torch

from g4b_b200.kernels import fa2
from helpers import assert_close, make_paged_case, make_ring_case, orc


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


def _oracle(case, layout, user_phase=None, o_init=None):
    q = case["q"]
    o = torch.zeros(q.shape) if o_init is None else o_init
    if layout == "paged":
        return orc.flash_attention(q, case["k_pool"], case["v_pool"], o, case["time"], user_phase, case["max_len"], 2,
                                   scale=1 / 16, block_tables=case["block_tables"], page_size=16)
    return orc.flash_attention(q, case["k"], case["v"], o, case["time"], user_phase, case["ctx_window"], 2, scale=1 / 16)


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
        assert_close(got, _oracle(case, layout), f"static scratch against the oracle, {layout}, {splits} splits")
    # and once more on the first inputs, now that the array holds the second call's partials
    assert_close(_static_call(first, cuda, 16, "paged"), _reference_call(first, cuda, 16, "paged").float(),
                 "static scratch, repeat")


@pytest.mark.gpu
def test_static_scratch_call_allocates_nothing(cuda):
    """Free device memory as the driver reports it is the same before and after calls of the
    entry point (inputs and outputs are made first, and the first call on the device, which
    looks up the array's address, is made before the reading)."""
    case = make_paged_case(73, lens=[2000, 900], H=8, G=2, dtype=torch.float16)
    q, kp, vp, bt, time = (case[n].to(cuda) for n in ("q", "k_pool", "v_pool", "block_tables", "time"))
    o = torch.zeros_like(q)
    call = lambda: fa2.decode_attention_static_scratch(q, kp, vp, o, time, None, case["max_len"], fa2.PHASE_DECODE,
                                                       scale=1 / 16, block_tables=bt, page_size=16, num_kv_splits=8)
    call()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    torch_before = torch.cuda.memory_allocated()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"free device memory moved by {free_before - free_after} bytes"
    assert torch.cuda.memory_allocated() == torch_before
    assert_close(o, _oracle(case, "paged"), "static scratch")


@pytest.mark.gpu
def test_static_scratch_auto_split_count_and_off_phase_slot(cuda):
    """No split count asked for, a window beyond 4096 and many slots: the reference's table
    says 8 splits, 8 x 260 x 8 = 16640 rows do not fit the 8192-row array, so the entry point
    drops to 3 and serves the batch.  One slot is off phase: its rows of the shared array keep
    whatever an earlier call left there, and its row of o must stay as it was."""
    B = 260
    case = make_ring_case(74, B=B, H=8, G=2, Tq=1, T=64, dtype=torch.float16, times=[64] * B, ctx_window=64)
    phase = torch.full((B,), 2, dtype=torch.uint8)
    phase[7] = 1
    q, k, v, time = (case[n].to(cuda) for n in ("q", "k", "v", "time"))
    o = torch.full(q.shape, 3.0, dtype=q.dtype, device=cuda)
    # ctx_window_size is the static bound the split policy looks at; the ring must be that long
    T = 8192
    kbig = torch.zeros(B, 2, T, 256, dtype=torch.float16, device=cuda)
    vbig = torch.zeros_like(kbig)
    kbig[:, :, :64], vbig[:, :, :64] = k, v
    fa2.decode_attention_static_scratch(q, kbig, vbig, o, time, phase.to(cuda), T, fa2.PHASE_DECODE, scale=1 / 16)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.full(q.shape, 3.0), case["time"], phase, 64, 2,
                               scale=1 / 16)
    assert_close(o, want, "static scratch, auto split count")
    assert bool((o[7] == 3.0).all()), "the off-phase slot's output was touched"


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
