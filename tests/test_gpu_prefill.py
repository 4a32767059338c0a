"""Flash-attention prefill (tcgen05 kernel) on the GPU, through the C ABI, against the oracle
and the reference-generated golden fixtures.  Tolerance: |a-b| <= 2e-3 + 1e-2 |b|."""
from pathlib import Path

import numpy as np
import pytest
import torch

from g4b_b200.kernels import fa2
from g4b_b200.kernels.add_kv_to_cache import add_kv_to_cache
from helpers import assert_close, make_ring_case, orc, randn

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


def run(case, cuda, *, scale=1 / 16, stage=fa2.STAGE_CAUSAL, sliding_window=None, phase_t=None,
        o_dtype=None, o_init=None, phase=fa2.PHASE_PREFILL):
    q_phys, k, v, time = (case[n].to(cuda) for n in ("q_phys", "k", "v", "time"))
    B, Tq, H, D = q_phys.shape
    o_phys = (torch.zeros(B, Tq, H, D, dtype=o_dtype or q_phys.dtype, device=cuda)
              if o_init is None else o_init.to(cuda))
    ph = None if phase_t is None else phase_t.to(cuda)
    fa2.flash_attention(q_phys.permute(0, 2, 1, 3), k, v, o_phys.permute(0, 2, 1, 3), time, ph,
                        case["ctx_window"], phase, stage=stage, scale=scale, sliding_window=sliding_window)
    return o_phys.permute(0, 2, 1, 3).cpu()


def oracle(case, *, scale=1 / 16, stage=fa2.STAGE_CAUSAL, sliding_window=None, phase_t=None, o_init=None,
           phase=fa2.PHASE_PREFILL):
    o0 = torch.zeros_like(case["q"], dtype=torch.float32) if o_init is None else o_init.permute(0, 2, 1, 3)
    return orc.flash_attention(case["q"], case["k"], case["v"], o0, case["time"], phase_t, case["ctx_window"],
                               phase, stage=stage, scale=scale, sliding_window=sliding_window)


@pytest.mark.parametrize("name", ["prefill_causal", "prefill_causal_unscaled", "prefill_swa", "prefill_chunked"])
def test_prefill_matches_reference_golden(cuda, name):
    """The committed outputs of the reference's LayerKVCache, reproduced by append + attention
    on the GPU (fp16; the fixture inputs are fp16-exact)."""
    z = np.load(GOLD / f"{name}.npz")
    q = torch.from_numpy(z["q"])          # [H,Tq,D] fp16
    k_all, v_all = torch.from_numpy(z["k_all"]), torch.from_numpy(z["v_all"])
    H, Tq, D = q.shape
    G, n_all, _ = k_all.shape
    is_swa, window = bool(z["is_swa"]), int(z["window"])
    T = 64
    k_cache = torch.zeros(1, G, T, D, dtype=torch.float16, device=cuda)
    v_cache = torch.zeros_like(k_cache)
    off = torch.zeros(1, dtype=torch.int32, device=cuda)
    add_kv_to_cache(k_all[None].to(cuda), k_cache, off, 1e-6)
    add_kv_to_cache(v_all[None].to(cuda), v_cache, off, 1e-6)
    o = torch.zeros(1, H, Tq, D, dtype=torch.float16, device=cuda)
    time = torch.tensor([n_all], dtype=torch.int32, device=cuda)
    ctx_window = min(T, window + Tq - 1) if is_swa else T
    fa2.flash_attention(q[None].to(cuda), k_cache, v_cache, o, time, None, ctx_window, 1,
                        scale=float(z["scale"]), sliding_window=window if is_swa else None)
    assert_close(o[0].cpu(), torch.from_numpy(z["out"]), name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,G,Tq,T", [(2, 8, 2, 256, 1024), (1, 16, 4, 128, 512), (2, 4, 2, 200, 333)])
def test_prefill_chunk_over_ring_cache(cuda, dtype, B, H, G, Tq, T):
    """A prefill chunk attending to a longer (for odd slots: wrapped) ring cache --
    tests/compare_scripts/test_fa2.py:61-64 scaled down, incl. a ragged Tq and an odd T."""
    case = make_ring_case(40, B=B, H=H, G=G, Tq=Tq, T=T, dtype=dtype,
                          times=[T if b % 2 == 0 else T + 17 for b in range(B)])
    assert_close(run(case, cuda), oracle(case), "prefill over ring")


def test_prefill_reference_scale(cuda):
    case = make_ring_case(41, B=1, H=8, G=2, Tq=256, T=256, dtype=torch.float16)
    assert_close(run(case, cuda, scale=1.0), oracle(case, scale=1.0), "prefill scale 1")


@pytest.mark.parametrize("Tq", [1, 37, 128, 129, 640])
def test_prefill_fresh_causal_lengths(cuda, Tq):
    """Whole-prompt prefill into an empty cache (time == Tq), ragged lengths incl. Tq == 1 run
    through the prefill kernel."""
    case = make_ring_case(42, B=2, H=8, G=2, Tq=Tq, T=640, dtype=torch.bfloat16, times=[Tq, Tq])
    q_phys, k, v, time = (case[n].to(cuda) for n in ("q_phys", "k", "v", "time"))
    o_phys = torch.zeros_like(q_phys)
    import ctypes
    from g4b_b200 import _cabi
    a = fa2._attn_args(q_phys.permute(0, 2, 1, 3), k, v, o_phys.permute(0, 2, 1, 3), time, None, 640, 1,
                       None, None, None, fa2.STAGE_CAUSAL, 1 / 16, None, None, 16, None)
    _cabi.check(_cabi.load().g4b_attn_prefill(ctypes.byref(a), ctypes.c_void_p(_cabi.current_stream())))
    assert_close(o_phys.permute(0, 2, 1, 3).cpu(), oracle(case), f"fresh prefill Tq={Tq}")


@pytest.mark.parametrize("Tq,W", [(1024, 128), (1024, 100), (700, 512), (384, 1)])
def test_prefill_sliding_window_per_query(cuda, Tq, W):
    """Per-query window (scripts/reference_impl.py:440-441): key visible iff 0 <= q_pos - k_pos < W."""
    case = make_ring_case(43, B=2, H=8, G=2, Tq=Tq, T=Tq, dtype=torch.bfloat16, times=[Tq, Tq])
    assert_close(run(case, cuda, sliding_window=W), oracle(case, sliding_window=W), f"swa W={W}")


def test_prefill_chunk_shared_window(cuda):
    """The reference kernel's own SWA form: the cache exposes W + t - 1 keys and every query
    of the chunk sees back to the first of them (fa2.py:52-67)."""
    Tq, W, T = 128, 256, 512
    case = make_ring_case(44, B=2, H=8, G=2, Tq=Tq, T=T, dtype=torch.float16, ctx_window=W + Tq - 1,
                          times=[W + Tq - 1, 2000])
    assert_close(run(case, cuda), oracle(case), "chunk-shared window")


def test_prefill_stage_full(cuda):
    # test_fa2.py:78: non-causal, Tq == Tcache == window
    case = make_ring_case(45, B=2, H=16, G=4, Tq=256, T=256, dtype=torch.float16, times=[256, 256])
    assert_close(run(case, cuda, stage=fa2.STAGE_FULL), oracle(case, stage=fa2.STAGE_FULL), "stage full")


def test_prefill_skips_slots_off_phase_and_f32_output(cuda):
    case = make_ring_case(46, B=3, H=8, G=2, Tq=128, T=256, dtype=torch.bfloat16, times=[256, 200, 128])
    phase_t = torch.tensor([1, 2, 1], dtype=torch.uint8)
    gen = torch.Generator().manual_seed(2)
    o_init = randn(gen, 3, 128, 8, 256)
    got = run(case, cuda, phase_t=phase_t, o_init=o_init)
    want = oracle(case, phase_t=phase_t, o_init=o_init)
    assert_close(got, want, "phase skip + f32 o")
    assert torch.equal(got[1], o_init.permute(0, 2, 1, 3)[1])


def test_prefill_window_tail_rows_may_hold_garbage(cuda):
    """Cache rows past the context are never multiplied in: fill them with NaN."""
    case = make_ring_case(47, B=1, H=8, G=2, Tq=100, T=512, dtype=torch.bfloat16, times=[300])
    case["k"][:, :, 300:] = float("nan")
    case["v"][:, :, 300:] = float("nan")
    got = run(case, cuda)
    case["k"][:, :, 300:] = 0
    case["v"][:, :, 300:] = 0
    assert_close(got, oracle(case), "garbage tail")


def test_prefill_full_size_rows(cuda):
    """Benchmark shape (B4 S8192 H8 G2 D256 bf16, causal, scale 1/16): sampled rows against
    the oracle, and invariance of every row to what lies after it in the cache."""
    gen = torch.Generator().manual_seed(48)
    B, S, H, G, D = 4, 8192, 8, 2, 256
    q_phys = randn(gen, B, S, H, D, dtype=torch.bfloat16)
    k = randn(gen, B, G, S, D, dtype=torch.bfloat16)
    v = randn(gen, B, G, S, D, dtype=torch.bfloat16)
    time = torch.full((B,), S, dtype=torch.int32)
    qd, kd, vd = q_phys.to(cuda), k.to(cuda), v.to(cuda)
    o = torch.zeros_like(qd)
    fa2.flash_attention(qd.permute(0, 2, 1, 3), kd, vd, o.permute(0, 2, 1, 3), time.to(cuda), None, S, 1, scale=1 / 16)
    got = o.permute(0, 2, 1, 3).cpu()
    rows = [0, 1, 127, 128, 129, 4095, 4096, 5000, 8190, 8191]
    for b in range(B):
        for r in rows:
            want = orc.attention_core(q_phys[b, r:r + 1].permute(1, 0, 2), k[b, :, :r + 1], v[b, :, :r + 1], scale=1 / 16)
            assert_close(got[b, :, r:r + 1], want, f"b={b} row={r}")
    # causality: scrambling keys after position 4096 leaves rows <= 4096 bit-identical
    kd[:, :, 4097:] = torch.flip(kd[:, :, 4097:], dims=[2])
    vd[:, :, 4097:] = -vd[:, :, 4097:]
    o2 = torch.zeros_like(qd)
    fa2.flash_attention(qd.permute(0, 2, 1, 3), kd, vd, o2.permute(0, 2, 1, 3), time.to(cuda), None, S, 1, scale=1 / 16)
    assert torch.equal(o2[:, :4097], o[:, :4097])
    assert not torch.equal(o2[:, 4097:], o[:, 4097:])


def test_prefill_sliding_window_full_size_rows(cuda):
    """Config shape B2 S32768 W512: sampled rows, each against its own 512-key window."""
    gen = torch.Generator().manual_seed(49)
    B, S, H, G, D, W = 2, 32768, 8, 2, 256, 512
    q_phys = randn(gen, B, S, H, D, dtype=torch.bfloat16)
    k = randn(gen, B, G, S, D, dtype=torch.bfloat16)
    v = randn(gen, B, G, S, D, dtype=torch.bfloat16)
    time = torch.full((B,), S, dtype=torch.int32)
    qd = q_phys.to(cuda)
    o = torch.zeros_like(qd)
    fa2.flash_attention(qd.permute(0, 2, 1, 3), k.to(cuda), v.to(cuda), o.permute(0, 2, 1, 3), time.to(cuda), None,
                        S, 1, scale=1 / 16, sliding_window=W)
    got = o.permute(0, 2, 1, 3).cpu()
    for b in range(B):
        for r in [0, 5, 511, 512, 513, 1000, 16384, 32767]:
            lo = max(0, r - W + 1)
            want = orc.attention_core(q_phys[b, r:r + 1].permute(1, 0, 2), k[b, :, lo:r + 1], v[b, :, lo:r + 1], scale=1 / 16)
            assert_close(got[b, :, r:r + 1], want, f"b={b} row={r}")


# ------------------------------------------------------------------------------------------
# prefill over a paged cache (not in the reference: block tables + 16-token pages)
# ------------------------------------------------------------------------------------------
def make_paged_prefill_case(seed, *, times, Tq, H, G, page_size=16, dtype=torch.bfloat16, poison=False):
    from helpers import make_paged_case
    case = make_paged_case(seed, lens=times, H=H, G=G, dtype=dtype, page_size=page_size)
    gen = torch.Generator().manual_seed(seed + 1)
    B = len(times)
    case["q_phys"] = randn(gen, B, Tq, H, 256, dtype=dtype)
    case["q"] = case["q_phys"].permute(0, 2, 1, 3)
    if poison:   # rows past each sequence's length hold NaN: they must never be multiplied in
        for b, n in enumerate(times):
            last = int(case["block_tables"][b, (n - 1) // page_size])
            r = n % page_size
            if r:
                case["k_pool"][last, :, r:] = float("nan")
                case["v_pool"][last, :, r:] = float("nan")
    return case


def run_paged_prefill(case, cuda, *, ctx_window=None, sliding_window=None, stage=fa2.STAGE_CAUSAL):
    q_phys = case["q_phys"].to(cuda)
    o_phys = torch.zeros_like(q_phys)
    fa2.flash_attention(q_phys.permute(0, 2, 1, 3), case["k_pool"].to(cuda), case["v_pool"].to(cuda),
                        o_phys.permute(0, 2, 1, 3), case["time"].to(cuda), None, ctx_window or case["max_len"], 1,
                        scale=1 / 16, sliding_window=sliding_window, block_tables=case["block_tables"].to(cuda),
                        page_size=case["page_size"], stage=stage)
    return o_phys.permute(0, 2, 1, 3).cpu()


def oracle_paged_prefill(case, *, ctx_window=None, sliding_window=None, stage=fa2.STAGE_CAUSAL):
    kp = torch.nan_to_num(case["k_pool"].float(), nan=0.0)
    vp = torch.nan_to_num(case["v_pool"].float(), nan=0.0)
    return orc.flash_attention(case["q"], kp, vp, torch.zeros_like(case["q"], dtype=torch.float32), case["time"], None,
                               ctx_window or case["max_len"], 1, stage=stage, scale=1 / 16,
                               sliding_window=sliding_window, block_tables=case["block_tables"],
                               page_size=case["page_size"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("times,Tq", [([128, 300, 1000], 128), ([200, 200], 200), ([640, 37 + 256, 513], 256)])
def test_prefill_paged_chunk(cuda, dtype, times, Tq):
    """The last Tq tokens of ragged contexts attend through shuffled block tables; partial
    last pages hold NaN beyond the context."""
    case = make_paged_prefill_case(60, times=times, Tq=Tq, H=8, G=2, dtype=dtype, poison=True)
    assert_close(run_paged_prefill(case, cuda), oracle_paged_prefill(case), "paged prefill")


def test_prefill_paged_windows_and_page_64(cuda):
    case = make_paged_prefill_case(61, times=[1000, 777], Tq=384, H=16, G=4, page_size=64, dtype=torch.float16)
    for kw in (dict(sliding_window=200), dict(ctx_window=500), dict(ctx_window=640, sliding_window=100),
               dict(stage=fa2.STAGE_FULL)):
        assert_close(run_paged_prefill(case, cuda, **kw), oracle_paged_prefill(case, **kw), f"paged prefill {kw}")


def test_prefill_paged_bad_table_entry_is_reported(cuda):
    from g4b_b200 import _cabi
    case = make_paged_prefill_case(62, times=[256], Tq=128, H=8, G=2)
    case["block_tables"][0, 3] = 10 ** 6
    got = run_paged_prefill(case, cuda)
    assert torch.isfinite(got).all()
    assert _cabi.device_status() == 0x309


def test_prefill_paged_equals_ring(cuda):
    """Same keys through a ring cache and through pages: identical outputs."""
    case = make_paged_prefill_case(63, times=[512, 512], Tq=512, H=8, G=2, dtype=torch.bfloat16)
    paged = run_paged_prefill(case, cuda)
    k = torch.stack([orc.gather_pages(case["k_pool"], case["block_tables"][b], 512, 16) for b in range(2)])
    v = torch.stack([orc.gather_pages(case["v_pool"], case["block_tables"][b], 512, 16) for b in range(2)])
    ring = dict(q_phys=case["q_phys"], q=case["q"], k=k.contiguous(), v=v.contiguous(), time=case["time"], ctx_window=512)
    assert torch.equal(run(ring, cuda), paged)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_prefill_long_contexts_use_the_long_item_kernel(cuda, dtype):
    """Contexts of several thousand keys select the long-item variant of the pair kernel (the
    small cases above all run the short-item one): chunked prefill at the end of paged
    contexts, and of a ring cache that wraps."""
    case = make_paged_prefill_case(64, times=[4500, 3333], Tq=256, H=8, G=2, dtype=dtype, poison=True)
    assert_close(run_paged_prefill(case, cuda), oracle_paged_prefill(case), "paged, long contexts")
    ring = make_ring_case(65, B=2, H=8, G=2, Tq=384, T=4100, dtype=dtype, times=[4100 + 777, 3000])
    assert_close(run(ring, cuda), oracle(ring), "ring, long contexts")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,G,Tq,T", [(2, 8, 2, 200, 333), (1, 3, 3, 129, 129), (2, 8, 2, 384, 4200)])
def test_prefill_accepts_f32_q_and_o(cuda, dtype, B, H, G, Tq, T):
    """The engine's scratchpad types (g4b/models/gemma4e.py:30-32): q and o fp32, caches 16-bit.
    q is rounded to the cache type on load; pair and one-CTA forms, short- and long-item kernels."""
    case = make_ring_case(70 + Tq, B=B, H=H, G=G, Tq=Tq, T=T, dtype=dtype)
    gen = torch.Generator().manual_seed(71)
    q32 = randn(gen, B, Tq, H, 256)                                   # not representable in 16 bits
    case32 = dict(case, q_phys=q32, q=q32.permute(0, 2, 1, 3))
    want = oracle(dict(case, q=q32.to(dtype).float().permute(0, 2, 1, 3)))
    got = run(case32, cuda, o_dtype=torch.float32)
    assert got.dtype == torch.float32
    assert_close(got, want, "f32 q, f32 o")
    got16 = run(case32, cuda, o_dtype=dtype)
    assert_close(got16, want, "f32 q, 16-bit o")


def run_split(case, cuda, *, splits, max_splits=8, sliding_window=None, stage=fa2.STAGE_CAUSAL, o_dtype=None):
    q_phys, k, v, time = (case[n].to(cuda) for n in ("q_phys", "k", "v", "time"))
    B, Tq, H, D = q_phys.shape
    o_phys = torch.zeros(B, Tq, H, D, dtype=o_dtype or q_phys.dtype, device=cuda)
    po = torch.full((max_splits, B, H, Tq, D), float("nan"), device=cuda)      # whatever is read must have been written
    pl = torch.full((max_splits, B, H, Tq), float("nan"), device=cuda)
    pm = torch.full((max_splits, B, H, Tq), float("nan"), device=cuda)
    fa2.flash_attention(q_phys.permute(0, 2, 1, 3), k, v, o_phys.permute(0, 2, 1, 3), time, None, case["ctx_window"], 1,
                        po, pl, pm, stage=stage, scale=1 / 16, sliding_window=sliding_window, num_kv_splits=splits)
    return o_phys.permute(0, 2, 1, 3).cpu(), (po, pl, pm)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("splits", [None, 2, 5, 8])
def test_prefill_split_kv_chunk(cuda, dtype, splits):
    """A chunk of 200 rows at the end of contexts of a few thousand keys, with the key range
    of every work item cut into pieces (forced counts, and the count the launcher picks when it
    is given partial buffers): same answer as the oracle, and as the unsplit kernel."""
    case = make_ring_case(80, B=2, H=8, G=2, Tq=200, T=3000, dtype=dtype, times=[3000 + 40, 2222])
    want = oracle(case)
    got, (po, pl, pm) = run_split(case, cuda, splits=splits)
    assert_close(got, want, f"split-KV prefill, {splits} splits")
    assert_close(got, run(case, cuda).float(), "split vs unsplit")


def test_prefill_split_kv_empty_ranges_windows_and_f32(cuda):
    """More pieces than some items have tiles (early query tiles of a causal prefill see one or
    two tiles: their later pieces are empty), a sliding window, STAGE_FULL, f32 output, and a
    slot off phase whose rows must keep their content."""
    case = make_ring_case(81, B=2, H=4, G=2, Tq=640, T=640, dtype=torch.bfloat16, times=[640, 640])
    for kw in (dict(), dict(sliding_window=200), dict(stage=fa2.STAGE_FULL)):
        got, _ = run_split(case, cuda, splits=4, o_dtype=torch.float32, **kw)
        assert_close(got, oracle(case, **kw), f"split-KV {kw}")
    q_phys, k, v, time = (case[n].to(cuda) for n in ("q_phys", "k", "v", "time"))
    o = torch.full((2, 640, 4, 256), 3.0, dtype=torch.bfloat16, device=cuda)
    ph = torch.tensor([1, 2], dtype=torch.uint8, device=cuda)
    po = torch.zeros(4, 2, 4, 640, 256, device=cuda); pl = torch.zeros(4, 2, 4, 640, device=cuda); pm = torch.zeros(4, 2, 4, 640, device=cuda)
    fa2.flash_attention(q_phys.permute(0, 2, 1, 3), k, v, o.permute(0, 2, 1, 3), time, ph, 640, 1, po, pl, pm, scale=1 / 16,
                        num_kv_splits=4)
    assert_close(o[0].permute(1, 0, 2).cpu(), oracle(case)[0], "slot in phase")
    assert (o[1] == 3.0).all()


def test_prefill_split_kv_paged_long_context(cuda):
    """The shape split-KV is for: one request, 256 new rows, tens of thousands of keys in pages."""
    case = make_paged_prefill_case(82, times=[20000], Tq=256, H=16, G=4, dtype=torch.float16)
    q_phys = case["q_phys"].to(cuda)
    o_phys = torch.zeros_like(q_phys)
    S = 8
    po = torch.empty(S, 1, 16, 256, 256, device=cuda); pl = torch.empty(S, 1, 16, 256, device=cuda); pm = torch.empty(S, 1, 16, 256, device=cuda)
    fa2.flash_attention(q_phys.permute(0, 2, 1, 3), case["k_pool"].to(cuda), case["v_pool"].to(cuda), o_phys.permute(0, 2, 1, 3),
                        case["time"].to(cuda), None, case["max_len"], 1, po, pl, pm, scale=1 / 16,
                        block_tables=case["block_tables"].to(cuda), page_size=case["page_size"])
    assert_close(o_phys.permute(0, 2, 1, 3), oracle_paged_prefill(case), "paged split-KV prefill")
    assert torch.isfinite(pm[:4]).any()      # the launcher did split (16 pair items on 74 workers)


def test_prefill_ignores_f16_partials(cuda):
    """The engine's decode workspace is f16 (gemma4e.py:819): handed to a prefill call it is
    left alone and the chunk runs unsplit; asking for a split count with it is an error."""
    case = make_ring_case(83, B=1, H=8, G=2, Tq=128, T=2048, dtype=torch.float16)
    q_phys, k, v, time = (case[n].to(cuda) for n in ("q_phys", "k", "v", "time"))
    o = torch.zeros_like(q_phys)
    po = torch.full((4, 1, 8, 128, 256), 9.0, dtype=torch.float16, device=cuda)
    pl = torch.full((4, 1, 8, 128), 9.0, device=cuda); pm = torch.full((4, 1, 8, 128), 9.0, device=cuda)
    fa2.flash_attention(q_phys.permute(0, 2, 1, 3), k, v, o.permute(0, 2, 1, 3), time, None, 2048, 1, po, pl, pm, scale=1 / 16)
    assert_close(o.permute(0, 2, 1, 3), oracle(case), "unsplit with f16 partials present")
    assert (po == 9.0).all() and (pl == 9.0).all()
    with pytest.raises(ValueError):
        fa2.flash_attention(q_phys.permute(0, 2, 1, 3), k, v, o.permute(0, 2, 1, 3), time, None, 2048, 1, po, pl, pm,
                            scale=1 / 16, num_kv_splits=4)


def test_sliding_window_unit_of_a_query_range_split(cuda):
    """The unit a rank gets when the query range of a (request, kv head) pair is halved over
    GPUs (g4b_b200.dist.shard_prefill_units at 8 GPUs on the sliding-window benchmark): 4 query
    heads, 1 kv head, the second half of 32768 queries over its own keys plus the 511 before it
    (16895 keys, not a multiple of the tile).  Sampled rows against the oracle."""
    from g4b_b200.dist import shard_prefill_units

    (r, g, q_lo, q_hi, k_lo), = shard_prefill_units(2, 2, 32768, 8, 1, 512)
    assert (q_lo, q_hi, k_lo) == (16384, 32768, 16384 - 511)
    Tq, Tk, H, D, W = q_hi - q_lo, q_hi - k_lo, 4, 256, 512
    gen = torch.Generator(device=cuda).manual_seed(12)
    q = torch.randn(1, Tq, H, D, generator=gen, device=cuda).to(torch.bfloat16)
    k = torch.randn(1, 1, Tk, D, generator=gen, device=cuda).to(torch.bfloat16)
    v = torch.randn(1, 1, Tk, D, generator=gen, device=cuda).to(torch.bfloat16)
    o = torch.zeros_like(q)
    time = torch.tensor([Tk], dtype=torch.int32, device=cuda)
    fa2.flash_attention(q.permute(0, 2, 1, 3), k, v, o.permute(0, 2, 1, 3), time, None, Tk, fa2.PHASE_PREFILL,
                        scale=1 / 16, sliding_window=W)
    kc, vc = k[0].float().cpu(), v[0].float().cpu()
    for row in (0, 1, 127, 128, 511, 512, 8191, Tq - 2, Tq - 1):
        pos = Tk - Tq + row
        want = orc.attention_core(q[0, row:row + 1].permute(1, 0, 2).float().cpu(), kc[:, :pos + 1], vc[:, :pos + 1],
                                  scale=1 / 16, sliding_window=W)
        assert_close(o[0, row:row + 1].permute(1, 0, 2), want, f"row {row}")


@pytest.mark.parametrize("layout", ["rows_padded", "heads_padded"])
def test_prefill_output_view_leaves_its_surroundings_alone(cuda, layout):
    """The output tile leaves through TMA boxes of 32 rows x 64 columns: a ragged Tq (200 = six
    boxes and a quarter) written into a view of a larger buffer must not touch the rows past Tq
    of a (slot, head), nor the padding between heads."""
    B, H, G, Tq, T, D = 2, 8, 2, 200, 512, 256
    case = make_ring_case(41, B=B, H=H, G=G, Tq=Tq, T=T, dtype=torch.bfloat16, times=[T, T - 100])
    q_phys, k, v, time = (case[n].to(cuda) for n in ("q_phys", "k", "v", "time"))
    if layout == "rows_padded":
        big = torch.full((B, H, Tq + 56, D), 7.0, dtype=torch.bfloat16, device=cuda)     # [B,H,rows,D], 56 spare rows per head
        o = big[:, :, :Tq]
        spare = big[:, :, Tq:]
    else:
        big = torch.full((B, Tq, H + 3, D), 7.0, dtype=torch.bfloat16, device=cuda)      # [B,rows,heads,D], 3 spare heads per row
        o = big[:, :, :H].permute(0, 2, 1, 3)
        spare = big[:, :, H:]
    fa2.flash_attention(q_phys.permute(0, 2, 1, 3), k, v, o, time, None, case["ctx_window"], fa2.PHASE_PREFILL, scale=1 / 16)
    assert_close(o.cpu(), oracle(case), "output view")
    assert bool((spare == 7.0).all()), "the kernel wrote outside the output view"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_sliding_window_items_with_wildly_different_score_scales(cuda, dtype):
    """Short items start from the reference maximum the same row ended the worker's previous
    item with.  Heads and positions whose scores differ by orders of magnitude (a guess far too
    low, far too high, and rows whose first tile shows them no key at all) must give the same
    output as the oracle: 256 work items over 74 workers, so every worker carries a guess
    through several items."""
    gen = torch.Generator().manual_seed(53)
    B, S, H, G, D, W = 1, 4096, 16, 2, 256, 300
    q_phys = randn(gen, B, S, H, D, dtype=torch.float32)
    k = randn(gen, B, G, S, D, dtype=dtype)
    v = randn(gen, B, G, S, D, dtype=dtype)
    # per-head factors spanning 1e-2 .. 2e2 (scores up to ~ +-300 in log2 units after the 1/16),
    # and per-position stripes of 128 rows that are almost silent
    head_gain = torch.tensor([0.01, 200.0, 1.0, 60.0, 0.1, 120.0, 3.0, 0.02, 150.0, 0.5, 30.0, 0.01, 90.0, 1.0, 0.05, 180.0])
    q_phys = q_phys * head_gain[None, None, :, None]
    stripe = ((torch.arange(S) // 128) % 3 == 1).float() * 0.999
    q_phys = (q_phys * (1.0 - stripe)[None, :, None, None]).to(dtype)
    time = torch.full((B,), S, dtype=torch.int32)
    qd = q_phys.to(cuda)
    o = torch.zeros_like(qd)
    fa2.flash_attention(qd.permute(0, 2, 1, 3), k.to(cuda), v.to(cuda), o.permute(0, 2, 1, 3), time.to(cuda), None,
                        S, 1, scale=1 / 16, sliding_window=W)
    got = o.permute(0, 2, 1, 3).cpu()
    assert bool(torch.isfinite(got.float()).all())
    rows = [0, 1, 127, 128, 129, 255, 256, 299, 300, 301, 383, 384, 1000, 2047, 2048, 2175, 2176, 3000, 4094, 4095]
    for r in rows:
        lo = max(0, r - W + 1)
        want = orc.attention_core(q_phys[0, r:r + 1].permute(1, 0, 2), k[0, :, lo:r + 1], v[0, :, lo:r + 1], scale=1 / 16)
        assert_close(got[0, :, r:r + 1], want, f"row={r}")



# ------------------------------------------------------------------------------------------
# head dim 128 (the kernel's tiles are 256 wide: the upper half is zero fill, never stored)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,G,Tq,T", [(2, 8, 2, 256, 1024), (1, 3, 3, 200, 333), (2, 4, 2, 130, 517)])
def test_prefill_head_dim_128_over_ring_cache(cuda, dtype, B, H, G, Tq, T):
    """CTA pairs and the one-CTA form (odd head count), wrapped rings (the tile that crosses the
    end of the ring is staged by ordinary loads), ragged Tq; the memory after every output row
    (the next head's row) must stay as it was."""
    case = make_ring_case(60, B=B, H=H, G=G, Tq=Tq, T=T, D=128, dtype=dtype,
                          times=[T if b % 2 == 0 else T + 17 for b in range(B)])
    assert_close(run(case, cuda), oracle(case), "head dim 128 over ring")


def test_prefill_head_dim_128_windows_f32_and_full_stage(cuda):
    case = make_ring_case(61, B=2, H=8, G=2, Tq=384, T=384, D=128, dtype=torch.bfloat16, times=[384, 384])
    assert_close(run(case, cuda, sliding_window=100), oracle(case, sliding_window=100), "head dim 128, sliding window")
    assert_close(run(case, cuda, stage=fa2.STAGE_FULL), oracle(case, stage=fa2.STAGE_FULL), "head dim 128, full stage")
    assert_close(run(case, cuda, o_dtype=torch.float32), oracle(case), "head dim 128, f32 output")
    # f32 q (rounded to the cache type on load)
    q32 = case["q_phys"].float().to(cuda)
    o = torch.zeros(2, 384, 8, 128, dtype=torch.bfloat16, device=cuda)
    fa2.flash_attention(q32.permute(0, 2, 1, 3), case["k"].to(cuda), case["v"].to(cuda), o.permute(0, 2, 1, 3),
                        case["time"].to(cuda), None, 384, fa2.PHASE_PREFILL, scale=1 / 16)
    assert_close(o.permute(0, 2, 1, 3).cpu(), oracle(case), "head dim 128, f32 q")


def test_prefill_head_dim_128_paged_and_split(cuda):
    """Over a paged cache (16-row TMA boxes per page), and a short chunk over a long context
    with the key range split and merged."""
    from helpers import make_paged_case

    times, Tq, H, G = [640, 37 + 256, 513], 256, 8, 2
    case = make_paged_case(62, lens=times, H=H, G=G, D=128, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(63)
    q_phys = randn(gen, 3, Tq, H, 128, dtype=torch.bfloat16)
    o = torch.zeros_like(q_phys).to(cuda)
    fa2.flash_attention(q_phys.to(cuda).permute(0, 2, 1, 3), case["k_pool"].to(cuda), case["v_pool"].to(cuda),
                        o.permute(0, 2, 1, 3), case["time"].to(cuda), None, case["max_len"], 1, scale=1 / 16,
                        block_tables=case["block_tables"].to(cuda), page_size=16)
    want = orc.flash_attention(q_phys.permute(0, 2, 1, 3), case["k_pool"].float(), case["v_pool"].float(),
                               torch.zeros(3, H, Tq, 128), case["time"], None, case["max_len"], 1, scale=1 / 16,
                               block_tables=case["block_tables"], page_size=16)
    assert_close(o.permute(0, 2, 1, 3).cpu(), want, "head dim 128, paged")
    # split-KV chunk: B1 H8 G2, 128 rows over 4096 keys, 4 splits
    ring = make_ring_case(64, B=1, H=8, G=2, Tq=128, T=4096, D=128, dtype=torch.bfloat16, times=[4096])
    q, k, v, time = (ring[n].to(cuda) for n in ("q_phys", "k", "v", "time"))
    po = torch.empty(4, 1, 8, 128, 128, device=cuda)
    pl, pm = torch.empty(4, 1, 8, 128, device=cuda), torch.empty(4, 1, 8, 128, device=cuda)
    o2 = torch.zeros(1, 128, 8, 128, dtype=torch.bfloat16, device=cuda)
    fa2.flash_attention(q.permute(0, 2, 1, 3), k, v, o2.permute(0, 2, 1, 3), time, None, 4096, fa2.PHASE_PREFILL,
                        po, pl, pm, scale=1 / 16, num_kv_splits=4)
    assert_close(o2.permute(0, 2, 1, 3).cpu(), oracle(ring), "head dim 128, split-KV chunk")



@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_causal_items_with_wildly_different_score_scales(cuda, dtype):
    """The same for long (causal) items, whose first tile takes the general path when the
    carried maximum does not hold: 256 items over 74 workers, heads whose scores differ by
    orders of magnitude, stripes of almost silent rows."""
    gen = torch.Generator().manual_seed(54)
    B, S, H, G, D = 1, 4096, 16, 2, 256
    q_phys = randn(gen, B, S, H, D, dtype=torch.float32)
    k = randn(gen, B, G, S, D, dtype=dtype)
    v = randn(gen, B, G, S, D, dtype=dtype)
    head_gain = torch.tensor([150.0, 0.01, 60.0, 1.0, 0.02, 200.0, 0.1, 3.0, 0.5, 90.0, 0.01, 30.0, 180.0, 0.05, 1.0, 120.0])
    q_phys = q_phys * head_gain[None, None, :, None]
    stripe = ((torch.arange(S) // 128) % 3 == 2).float() * 0.999
    q_phys = (q_phys * (1.0 - stripe)[None, :, None, None]).to(dtype)
    time = torch.full((B,), S, dtype=torch.int32)
    qd = q_phys.to(cuda)
    o = torch.zeros_like(qd)
    fa2.flash_attention(qd.permute(0, 2, 1, 3), k.to(cuda), v.to(cuda), o.permute(0, 2, 1, 3), time.to(cuda), None,
                        S, 1, scale=1 / 16)
    got = o.permute(0, 2, 1, 3).cpu()
    assert bool(torch.isfinite(got.float()).all())
    for r in [0, 1, 63, 64, 127, 128, 129, 255, 256, 383, 384, 1000, 2047, 2048, 2175, 3000, 4094, 4095]:
        want = orc.attention_core(q_phys[0, r:r + 1].permute(1, 0, 2), k[0, :, :r + 1], v[0, :, :r + 1], scale=1 / 16)
        assert_close(got[0, :, r:r + 1], want, f"row={r}")
