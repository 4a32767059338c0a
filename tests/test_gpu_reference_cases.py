"""The case list of the reference's own attention comparison script
(tests/compare_scripts/test_fa2.py:51-79), run through the C ABI and checked against the
oracle: same shapes, same fp16 ring caches filled everywhere, same time_dim_sizes pattern
(ctx_window for even slots, ctx_window + 17 for odd ones, so that odd slots wrap the ring,
test_fa2.py:285-290), same split workspace sizes.  The script itself asserts nothing and
seeds nothing; the oracle is what pins the numbers."""
import pytest
import torch

from g4b_b200.kernels import fa2
from helpers import assert_close, make_ring_case, orc

pytestmark = pytest.mark.gpu

DECODE = [  # name, B, H, G, T, max_kv_splits (test_fa2.py:52-58; default workspace 4, :46)
    ("decode_gemma_w4096", 8, 16, 4, 4096, 4),
    ("decode_gemma_w8192", 4, 16, 4, 8192, 4),
    ("decode_gemma_w16384", 2, 16, 4, 16384, 4),
    ("decode_gemma_w32768", 1, 16, 4, 32768, 4),
    ("decode_gemma_w65536", 1, 16, 4, 65536, 64),
    ("decode_biggroup_w4096", 4, 32, 4, 4096, 4),
]
PREFILL = [  # name, B, H, G, Tq, T, stage (test_fa2.py:60-78)
    ("prefill_t128_w4096", 2, 16, 4, 128, 4096, fa2.STAGE_CAUSAL),
    ("prefill_t256_w4096", 1, 16, 4, 256, 4096, fa2.STAGE_CAUSAL),
    ("prefill_t256_w8192", 1, 16, 4, 256, 8192, fa2.STAGE_CAUSAL),
    ("prefill_t256_w65536", 1, 16, 4, 256, 65536, fa2.STAGE_CAUSAL),
    ("full_t256_w256", 2, 16, 4, 256, 256, fa2.STAGE_FULL),
]


@pytest.mark.parametrize("name,B,H,G,T,max_splits", DECODE)
def test_reference_decode_cases(cuda, name, B, H, G, T, max_splits):
    case = make_ring_case(900 + T // 1024 + H, B=B, H=H, G=G, Tq=1, T=T, dtype=torch.float16)
    q, k, v, time = (case[n].to(cuda) for n in ("q", "k", "v", "time"))
    o = torch.zeros(B, H, 1, 256, dtype=torch.float16, device=cuda)
    po = torch.empty(max_splits, B, H, 1, 256, dtype=torch.float16, device=cuda)     # f16 like the engine's (gemma4e.py:819)
    pl = torch.empty(max_splits, B, H, 1, device=cuda)
    pm = torch.empty(max_splits, B, H, 1, device=cuda)
    fa2.flash_attention(q, k, v, o, time, torch.full((B,), 2, dtype=torch.uint8, device=cuda), T, fa2.PHASE_DECODE,
                        po, pl, pm, scale=1 / 16)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.zeros(B, H, 1, 256), case["time"], None, T, 2,
                               scale=1 / 16)
    assert_close(o, want, name)


@pytest.mark.parametrize("name,B,H,G,Tq,T,stage", PREFILL)
def test_reference_prefill_cases(cuda, name, B, H, G, Tq, T, stage):
    case = make_ring_case(950 + T // 1024 + Tq, B=B, H=H, G=G, Tq=Tq, T=T, dtype=torch.float16)
    q_phys, k, v, time = (case[n].to(cuda) for n in ("q_phys", "k", "v", "time"))
    o_phys = torch.zeros_like(q_phys)
    fa2.flash_attention(q_phys.permute(0, 2, 1, 3), k, v, o_phys.permute(0, 2, 1, 3), time,
                        torch.full((B,), 1, dtype=torch.uint8, device=cuda), T, fa2.PHASE_PREFILL, stage=stage, scale=1 / 16)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.zeros(B, H, Tq, 256), case["time"], None, T, 1,
                               stage=stage, scale=1 / 16)
    assert_close(o_phys.permute(0, 2, 1, 3), want, name)


def test_reference_prefill_t65536_sampled_rows(cuda):
    """prefill_t65536_w65536 (B1 H16 G4, 35 TFLOP): sampled query rows against the oracle."""
    B, H, G, S = 1, 16, 4, 65536
    gen = torch.Generator(device=cuda).manual_seed(5)
    q = torch.randn(B, S, H, 256, generator=gen, device=cuda).to(torch.float16)
    k = torch.randn(B, G, S, 256, generator=gen, device=cuda).to(torch.float16)
    v = torch.randn(B, G, S, 256, generator=gen, device=cuda).to(torch.float16)
    o = torch.zeros_like(q)
    time = torch.full((B,), S, dtype=torch.int32, device=cuda)
    fa2.flash_attention(q.permute(0, 2, 1, 3), k, v, o.permute(0, 2, 1, 3), time, None, S, fa2.PHASE_PREFILL, scale=1 / 16)
    rows = [0, 1, 127, 128, 4095, 33333, 65534, 65535]
    kc, vc = k[0].float().cpu(), v[0].float().cpu()
    for r in rows:
        want = orc.attention_core(q[0, r:r + 1].permute(1, 0, 2).float().cpu(), kc[:, : r + 1], vc[:, : r + 1], scale=1 / 16)
        assert_close(o[0, r:r + 1].permute(1, 0, 2), want, f"row {r}")


@pytest.mark.parametrize("with_splits", [False, True])
def test_reference_head_dim_128_decode_case(cuda, with_splits):
    """decode_small_w1024 (B4 H8 G2 D128, test_fa2.py:52), with the script's time pattern (odd
    slots wrap the ring) and, as its grouped_split variant, a 4-split workspace."""
    B, H, G, T, D = 4, 8, 2, 1024, 128
    case = make_ring_case(917, B=B, H=H, G=G, Tq=1, T=T, D=D, dtype=torch.float16)
    q, k, v, time = (case[n].to(cuda) for n in ("q", "k", "v", "time"))
    o = torch.zeros(B, H, 1, D, dtype=torch.float16, device=cuda)
    parts = ()
    if with_splits:
        parts = (torch.empty(4, B, H, 1, D, dtype=torch.float16, device=cuda), torch.empty(4, B, H, 1, device=cuda),
                 torch.empty(4, B, H, 1, device=cuda))
    fa2.flash_attention(q, k, v, o, time, None, T, fa2.PHASE_DECODE, *parts, num_kv_splits=4 if with_splits else None)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.zeros(B, H, 1, D), case["time"], None, T, 2)
    assert_close(o, want, "decode_small_w1024")


def test_prefill_head_dim_512_is_refused(cuda):
    """The Tq > 1 kernel takes head dims 128 and 256; others must be refused, not computed."""
    q = torch.zeros(1, 8, 64, 512, dtype=torch.float16, device=cuda)
    k = torch.zeros(1, 2, 1024, 512, dtype=torch.float16, device=cuda)
    time = torch.full((1,), 1024, dtype=torch.int32, device=cuda)
    with pytest.raises(ValueError, match="head dim"):
        fa2.flash_attention(q, k, k.clone(), torch.zeros_like(q), time, None, 1024, fa2.PHASE_PREFILL)
