"""The device status word across launches: a bad block-table entry that one launch reports
must not change what later launches compute.

Nothing here faults: a table entry outside the pool is never followed (the kernel skips the
row and records a code), which is the behaviour under test."""
import pytest
import torch

from g4b_b200 import _cabi
from g4b_b200.kernels import fa2
from g4b_b200.kernels.add_kv_to_cache import add_kv_to_cache
from helpers import assert_close, make_paged_case, make_ring_case, orc

pytestmark = pytest.mark.gpu


def test_prefill_still_computes_after_an_append_reported_a_bad_table_entry(cuda):
    # 1. an append whose block table points outside the pool: skipped and reported (0x1xx)
    G, D, ps = 2, 256, 16
    pool = torch.zeros(4, G, ps, D, dtype=torch.float16, device=cuda)
    x = torch.ones(1, G, 3, D, dtype=torch.float16, device=cuda)
    bad_table = torch.tensor([[0, 99, 1]], dtype=torch.int32, device=cuda)       # page 99 of 4
    add_kv_to_cache(x, pool, torch.tensor([15], dtype=torch.int32, device=cuda), 1e-6, block_tables=bad_table,
                    page_size=ps)
    torch.cuda.synchronize()
    assert bool((pool[0, :, 15] == 1).all()), "the row that had a valid page was not written"
    assert float(pool[1:].abs().sum()) == 0, "a row was written through the bad entry"

    # 2. without anybody reading the status word: a prefill launch and a decode launch on good
    # inputs give the oracle's answers
    case = make_ring_case(91, B=2, H=8, G=2, Tq=192, T=256, dtype=torch.bfloat16)
    o = torch.zeros(2, 192, 8, 256, dtype=torch.bfloat16, device=cuda)
    fa2.flash_attention(case["q"].to(cuda), case["k"].to(cuda), case["v"].to(cuda), o.permute(0, 2, 1, 3),
                        case["time"].to(cuda), None, 256, fa2.PHASE_PREFILL, scale=1 / 16)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.zeros(2, 8, 192, 256), case["time"], None, 256, 1,
                               scale=1 / 16)
    assert_close(o.permute(0, 2, 1, 3), want, "prefill after a reported bad table entry")

    dcase = make_paged_case(92, lens=[700, 33], H=8, G=2, dtype=torch.float16)
    od = torch.zeros(2, 8, 1, 256, dtype=torch.float16, device=cuda)
    fa2.flash_attention(dcase["q"].to(cuda), dcase["k_pool"].to(cuda), dcase["v_pool"].to(cuda), od,
                        dcase["time"].to(cuda), None, dcase["max_len"], fa2.PHASE_DECODE, scale=1 / 16,
                        block_tables=dcase["block_tables"].to(cuda), page_size=16)
    wantd = orc.flash_attention(dcase["q"], dcase["k_pool"], dcase["v_pool"], torch.zeros(2, 8, 1, 256), dcase["time"],
                                None, dcase["max_len"], 2, scale=1 / 16, block_tables=dcase["block_tables"], page_size=16)
    assert_close(od, wantd, "decode after a reported bad table entry")

    # 3. the word still holds the FIRST code, the append's; reading clears it, and the library
    # call says so with G4B_ERR_DEVICE_WAIT
    import ctypes

    out = ctypes.c_int32(0)
    rc = _cabi.load().g4b_device_status(ctypes.c_void_p(_cabi.current_stream()), ctypes.byref(out))
    assert rc == -6 and (out.value & 0xf00) == 0x100, (rc, hex(out.value))
    assert "0x1" in _cabi.load().g4b_last_error_string().decode()
    assert _cabi.device_status() == 0


def test_prefill_reports_its_own_bad_table_entry_and_later_launches_run(cuda):
    """A bad entry met by the prefill kernel itself (0x309) is reported and skipped; the next
    prefill launch, on good tables, computes normally without the word having been read."""
    from helpers import randn

    page, Tq = 16, 128
    case = make_paged_case(93, lens=[Tq + 40], H=8, G=2, dtype=torch.bfloat16, page_size=page)
    gen = torch.Generator().manual_seed(93)
    q_phys = randn(gen, 1, Tq, 8, 256, dtype=torch.bfloat16)
    q = q_phys.to(cuda).permute(0, 2, 1, 3)
    kp, vp, time = case["k_pool"].to(cuda), case["v_pool"].to(cuda), case["time"].to(cuda)
    bad = case["block_tables"].clone()
    bad[0, 1] = kp.shape[0] + 7
    o = torch.zeros(1, Tq, 8, 256, dtype=torch.bfloat16, device=cuda)
    fa2.flash_attention(q, kp, vp, o.permute(0, 2, 1, 3), time, None, case["max_len"], fa2.PHASE_PREFILL, scale=1 / 16,
                        block_tables=bad.to(cuda), page_size=page)
    torch.cuda.synchronize()
    o2 = torch.zeros_like(o)
    fa2.flash_attention(q, kp, vp, o2.permute(0, 2, 1, 3), time, None, case["max_len"], fa2.PHASE_PREFILL, scale=1 / 16,
                        block_tables=case["block_tables"].to(cuda), page_size=page)
    want = orc.flash_attention(q_phys.permute(0, 2, 1, 3), case["k_pool"], case["v_pool"], torch.zeros(1, 8, Tq, 256),
                               case["time"], None, case["max_len"], 1, scale=1 / 16, block_tables=case["block_tables"],
                               page_size=page)
    assert_close(o2.permute(0, 2, 1, 3), want, "prefill after a prefill launch met a bad table entry")
    assert _cabi.device_status() == 0x309
