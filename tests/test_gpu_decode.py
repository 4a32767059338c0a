"""Single-token decode attention (+ split-KV combine) on the GPU, through the C ABI, against
the oracle.  Tolerance for f16/bf16 outputs: |a-b| <= 2e-3 + 1e-2 |b|."""
import pytest
import torch

from g4b_b200.kernels import fa2
from helpers import assert_close, make_paged_case, make_ring_case, orc, randn

pytestmark = pytest.mark.gpu


def run_ring(case, cuda, *, splits=None, max_splits=0, scale=1.0, phase_t=None, sliding_window=None,
             partial_dtype=torch.float32, o_init=None):
    q, k, v, time = (case[n].to(cuda) for n in ("q", "k", "v", "time"))
    B, H, Tq, D = q.shape
    o_phys = torch.zeros(B, Tq, H, D, dtype=q.dtype, device=cuda) if o_init is None else o_init.to(cuda)
    o = o_phys.permute(0, 2, 1, 3)
    po = pl = pm = None
    if max_splits:
        po = torch.full((max_splits, B, H, Tq, D), float("nan"), dtype=partial_dtype, device=cuda)
        pl = torch.full((max_splits, B, H, Tq), float("nan"), device=cuda)
        pm = torch.full((max_splits, B, H, Tq), float("nan"), device=cuda)
    ph = None if phase_t is None else phase_t.to(cuda)
    fa2.flash_attention(q, k, v, o, time, ph, case["ctx_window"], fa2.PHASE_DECODE, po, pl, pm,
                        scale=scale, sliding_window=sliding_window, num_kv_splits=splits)
    return o.cpu()


# shapes of tests/compare_scripts/test_fa2.py:51-59, cache lengths scaled down
@pytest.mark.parametrize("B,H,G,T", [(4, 8, 2, 1024), (2, 16, 4, 2048), (2, 32, 4, 512), (1, 8, 8, 300)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_decode_ring_single_split(cuda, B, H, G, T, dtype):
    case = make_ring_case(20, B=B, H=H, G=G, Tq=1, T=T, dtype=dtype)   # odd slots wrapped
    got = run_ring(case, cuda, scale=1 / 16)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.zeros_like(case["q"], dtype=torch.float32),
                               case["time"], None, case["ctx_window"], 2, scale=1 / 16)
    assert_close(got, want, "decode ring")


def test_decode_ring_reference_scale(cuda):
    """The reference applies no softmax scale (fa2.py:89): near one-hot rows, |o| up to ~4."""
    case = make_ring_case(21, B=2, H=8, G=2, Tq=1, T=1024, dtype=torch.float16)
    got = run_ring(case, cuda, scale=1.0)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.zeros_like(case["q"], dtype=torch.float32),
                               case["time"], None, 1024, 2, scale=1.0)
    assert_close(got, want, "decode scale 1")


@pytest.mark.parametrize("splits,max_splits", [(4, 4), (16, 16), (3, 8), (None, 16)])
@pytest.mark.parametrize("partial_dtype", [torch.float32, torch.float16])
def test_decode_ring_split_kv(cuda, splits, max_splits, partial_dtype):
    case = make_ring_case(22, B=3, H=8, G=2, Tq=1, T=8192, dtype=torch.float16)   # policy: 8 splits
    got = run_ring(case, cuda, splits=splits, max_splits=max_splits, scale=1 / 16, partial_dtype=partial_dtype)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.zeros_like(case["q"], dtype=torch.float32),
                               case["time"], None, 8192, 2, scale=1 / 16)
    assert_close(got, want, f"decode splits={splits}")


def test_decode_short_contexts_and_empty_splits(cuda):
    """Contexts shorter than one block and fewer blocks than splits (empty splits carry
    m=-inf, l=0)."""
    case = make_ring_case(23, B=6, H=8, G=2, Tq=1, T=256, dtype=torch.bfloat16, times=[1, 2, 15, 16, 17, 40])
    got = run_ring(case, cuda, splits=8, max_splits=8, scale=1 / 16)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.zeros_like(case["q"], dtype=torch.float32),
                               case["time"], None, 256, 2, scale=1 / 16)
    assert_close(got, want, "short contexts")


def test_decode_skips_slots_off_phase(cuda):
    case = make_ring_case(24, B=4, H=8, G=2, Tq=1, T=512, dtype=torch.float16)
    phase_t = torch.tensor([2, 1, 0, 2], dtype=torch.uint8)
    gen = torch.Generator().manual_seed(1)
    o_init = randn(gen, 4, 1, 8, 256, dtype=torch.float16)
    for splits, cap in ((None, 0), (4, 4)):
        got = run_ring(case, cuda, splits=splits, max_splits=cap, scale=1 / 16, phase_t=phase_t, o_init=o_init)
        want = orc.flash_attention(case["q"], case["k"], case["v"], o_init.permute(0, 2, 1, 3), case["time"],
                                   phase_t, 512, 2, scale=1 / 16)
        assert_close(got, want, "phase skip")
        assert torch.equal(got[1], o_init.permute(0, 2, 1, 3)[1]) and torch.equal(got[2], o_init.permute(0, 2, 1, 3)[2])


def test_decode_sliding_window_equals_windowed_cache(cuda):
    """Tq == 1: a per-query window W equals exposing only the last W keys."""
    case = make_ring_case(25, B=2, H=8, G=2, Tq=1, T=1024, dtype=torch.float16, times=[700, 1024])
    got = run_ring(case, cuda, scale=1 / 16, sliding_window=100)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.zeros_like(case["q"], dtype=torch.float32),
                               case["time"], None, 1024, 2, scale=1 / 16, sliding_window=100)
    assert_close(got, want, "decode sliding window")


def run_paged(case, cuda, *, splits=None, max_splits=0, scale=1 / 16, sliding_window=None, ctx_window=None):
    q, kp, vp, bt, time = (case[n].to(cuda) for n in ("q", "k_pool", "v_pool", "block_tables", "time"))
    B, H, Tq, D = q.shape
    o = torch.zeros_like(q)
    po = pl = pm = None
    if max_splits:
        po = torch.empty(max_splits, B, H, Tq, D, dtype=torch.float32, device=cuda)
        pl = torch.empty(max_splits, B, H, Tq, device=cuda)
        pm = torch.empty(max_splits, B, H, Tq, device=cuda)
    fa2.flash_attention(q, kp, vp, o, time, None, ctx_window or case["max_len"], fa2.PHASE_DECODE, po, pl, pm,
                        scale=scale, sliding_window=sliding_window, block_tables=bt, page_size=case["page_size"],
                        num_kv_splits=splits)
    return o.cpu(), (po, pl, pm)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("splits,cap", [(None, 0), (8, 8), (16, 16)])
def test_decode_paged_ragged(cuda, dtype, splits, cap):
    lens = [1, 15, 16, 17, 31, 1000, 4097, 2048]
    case = make_paged_case(30, lens=lens, H=8, G=2, dtype=dtype)
    got, _ = run_paged(case, cuda, splits=splits, max_splits=cap)
    want = orc.flash_attention(case["q"], case["k_pool"], case["v_pool"], torch.zeros_like(case["q"], dtype=torch.float32),
                               case["time"], None, case["max_len"], 2, scale=1 / 16,
                               block_tables=case["block_tables"], page_size=16)
    assert_close(got, want, "decode paged")


def test_decode_paged_page_size_64_and_window(cuda):
    case = make_paged_case(31, lens=[130, 64, 700], H=16, G=4, dtype=torch.float16, page_size=64)
    got, _ = run_paged(case, cuda, sliding_window=257)
    want = orc.flash_attention(case["q"], case["k_pool"], case["v_pool"], torch.zeros_like(case["q"], dtype=torch.float32),
                               case["time"], None, case["max_len"], 2, scale=1 / 16, sliding_window=257,
                               block_tables=case["block_tables"], page_size=64)
    assert_close(got, want, "paged page 64 + window")


def test_decode_paged_window_shorter_than_context(cuda):
    """A paged cache keeps absolute positions: ctx_window_size < context exposes the tail."""
    case = make_paged_case(36, lens=[1000, 300, 77], H=8, G=2, dtype=torch.float16)
    got, _ = run_paged(case, cuda, ctx_window=200, splits=4, max_splits=4)
    want = orc.flash_attention(case["q"], case["k_pool"], case["v_pool"], torch.zeros_like(case["q"], dtype=torch.float32),
                               case["time"], None, 200, 2, scale=1 / 16, block_tables=case["block_tables"], page_size=16)
    assert_close(got, want, "paged, window < context")


def test_decode_partials_have_reference_format(cuda):
    """Partials written for S splits merge, with the oracle's combine (fa2.py:618-626), to the
    unsplit answer; the GPU combine agrees with the oracle's on the same partials."""
    case = make_paged_case(32, lens=[3000, 555], H=8, G=2, dtype=torch.float16)
    q, kp, vp, bt, time = (case[n].to(cuda) for n in ("q", "k_pool", "v_pool", "block_tables", "time"))
    S = 12
    po = torch.empty(S, 2, 8, 1, 256, device=cuda)
    pl = torch.empty(S, 2, 8, 1, device=cuda)
    pm = torch.empty(S, 2, 8, 1, device=cuda)
    o = torch.zeros_like(q)
    fa2.attention_decode_partials(q, kp, vp, o, time, None, case["max_len"], 2, po, pl, pm, S, scale=1 / 16,
                                  block_tables=bt, page_size=16)
    want = orc.flash_attention(case["q"], case["k_pool"], case["v_pool"], torch.zeros(2, 8, 1, 256), case["time"], None,
                               case["max_len"], 2, scale=1 / 16, block_tables=case["block_tables"], page_size=16)
    merged = orc.combine_partials(po.cpu(), pl.cpu(), pm.cpu(), S)
    assert_close(merged, want, "oracle merge of GPU partials")
    o32 = torch.zeros(2, 8, 1, 256, device=cuda)
    fa2.combine_partials(po, pl, pm, o32, S)
    assert torch.allclose(o32.cpu(), merged, rtol=1e-5, atol=1e-6)


def test_combine_kernel_against_oracle(cuda):
    gen = torch.Generator().manual_seed(33)
    S, B, H, Tq, D = 7, 3, 8, 2, 256
    po = randn(gen, S, B, H, Tq, D)
    pl = torch.rand(S, B, H, Tq, generator=gen) + 0.1
    pm = randn(gen, S, B, H, Tq) * 4
    pm[2] = float("-inf"); pl[2] = 0; po[2] = 0    # an empty split
    want = orc.combine_partials(po, pl, pm, S)
    for odt in (torch.float32, torch.float16, torch.bfloat16):
        o = torch.zeros(B, H, Tq, D, dtype=odt, device=cuda)
        fa2.combine_partials(po.to(cuda), pl.to(cuda), pm.to(cuda), o, S)
        assert_close(o.cpu(), want, f"combine {odt}", abs_tol=1e-5 if odt == torch.float32 else 2e-3)


def test_decode_full_size_property(cuda):
    """At benchmark size (contexts up to 32768, 16-token pages): the answer does not depend on
    the split count, and matches the oracle on the longest and the shortest sequence."""
    gen = torch.Generator().manual_seed(34)
    lens = torch.randint(1024, 32769, (24,), generator=gen).tolist()
    lens[0], lens[1] = 32768, 1024
    case = make_paged_case(35, lens=lens, H=8, G=2, dtype=torch.float16)
    a, _ = run_paged(case, cuda, splits=None, max_splits=0)
    b_, _ = run_paged(case, cuda, splits=16, max_splits=16)
    c, _ = run_paged(case, cuda, splits=5, max_splits=8)
    assert_close(b_, a.float(), "16 splits vs 1"); assert_close(c, a.float(), "5 splits vs 1")
    for b in (0, 1):
        k = orc.gather_pages(case["k_pool"], case["block_tables"][b], lens[b], 16)
        v = orc.gather_pages(case["v_pool"], case["block_tables"][b], lens[b], 16)
        assert_close(a[b], orc.attention_core(case["q"][b], k, v, scale=1 / 16), f"seq {b}")


def test_decode_one_long_sequence_full_size(cuda):
    """One sequence of 131072 tokens (bf16, 16-token pages, shuffled table): the whole answer
    against the oracle, for the split counts the benchmark uses and for the merge kernels."""
    from g4b_b200.dist import PartialExchange

    case = make_paged_case(36, lens=[131072], H=8, G=2, dtype=torch.bfloat16, extra_pages=5)
    k = orc.gather_pages(case["k_pool"], case["block_tables"][0], 131072, 16)
    v = orc.gather_pages(case["v_pool"], case["block_tables"][0], 131072, 16)
    want = orc.attention_core(case["q"][0], k, v, scale=1 / 16)
    for splits in (16, 148):
        got, (po, pl, pm) = run_paged(case, cuda, splits=splits, max_splits=splits)
        assert_close(got[0], want, f"{splits} splits")
    # the same partials through the one-kernel cross-GPU merge (a world of one)
    from g4b_b200 import _cabi
    peers = [torch.zeros(_cabi.load().g4b_exchange_buffer_bytes(1, 8, 256) // 8, dtype=torch.int64, device=cuda)]
    ex = PartialExchange(8, 256, peers=peers, rank=0)
    o = torch.zeros(1, 8, 1, 256, dtype=torch.bfloat16, device=cuda)
    ex.combine(po, pl, pm, o, 148)
    assert_close(o[0].cpu(), want, "exchange merge of 148 splits")


@pytest.mark.parametrize("H,G", [(16, 1), (12, 1), (9, 3)])
def test_single_token_with_more_than_8_heads_per_kv_head(cuda, H, G):
    """Groups wider than the decode kernel's 8 query heads per kv head (and head counts that
    rule out the CTA-pair form) still answer at Tq = 1: the call takes the prefill kernel."""
    case = make_ring_case(37 + H, B=3, H=H, G=G, Tq=1, T=700, dtype=torch.bfloat16, times=[700, 717, 5])
    q, k, v, time = (case[n].to(cuda) for n in ("q", "k", "v", "time"))
    o = torch.zeros_like(q)
    fa2.flash_attention(q, k, v, o, time, None, 700, fa2.PHASE_DECODE, scale=1 / 16)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.zeros(3, H, 1, 256), case["time"], None, 700, 2,
                               scale=1 / 16)
    assert_close(o, want, f"H{H} G{G} at Tq 1")
