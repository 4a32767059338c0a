"""Seeded random sweeps over shapes and options, GPU through the C ABI against the oracle.
The hand-picked cases elsewhere cover the edges someone thought of; these cover combinations
nobody did: head counts that switch kernel forms, chunk sizes off the tile grid, contexts
shorter than the chunk's tile, windows, rings that wrap, pages, split counts, slots off phase."""
import random

import pytest
import torch

from g4b_b200.kernels import fa2
from helpers import assert_close, make_paged_case, make_ring_case, orc

pytestmark = pytest.mark.gpu

HEADS = [(8, 2), (4, 4), (16, 4), (6, 2), (3, 1), (2, 2), (12, 4), (5, 5)]


def _phase_vec(rng, B, phase):
    ph = [phase if rng.random() < 0.8 else rng.choice([0, 3 - phase]) for _ in range(B)]
    ph[0] = phase
    return torch.tensor(ph, dtype=torch.uint8)


@pytest.mark.parametrize("seed", range(24))
def test_random_prefill_ring(cuda, seed):
    rng = random.Random(1000 + seed)
    H, G = rng.choice(HEADS)
    B = rng.randint(1, 3)
    Tq = rng.choice([1, 2, 17, 64, 127, 128, 129, 200, 256, 300])
    T = Tq + rng.choice([0, 1, 15, 100, 333, 1000])
    ctx_window = rng.choice([T, max(Tq, T - rng.randint(0, T // 2))])
    dtype = rng.choice([torch.float16, torch.bfloat16])
    times = [rng.choice([ctx_window, ctx_window + rng.randint(1, 2 * T), max(Tq, ctx_window - rng.randint(0, ctx_window - Tq))])
             for _ in range(B)]
    case = make_ring_case(2000 + seed, B=B, H=H, G=G, Tq=Tq, T=T, dtype=dtype, times=times, ctx_window=ctx_window)
    stage = rng.choice([fa2.STAGE_CAUSAL, fa2.STAGE_CAUSAL, fa2.STAGE_FULL])
    sw = rng.choice([None, None, rng.randint(1, max(1, ctx_window))])
    scale = rng.choice([1.0 / 16, 1.0, 0.03])
    o_dtype = rng.choice([dtype, torch.float32])
    ph = _phase_vec(rng, B, 1)
    q_phys, k, v, time = (case[n].to(cuda) for n in ("q_phys", "k", "v", "time"))
    if rng.random() < 0.3:
        q_phys = q_phys.float()                     # the engine's f32 scratchpad
    o_phys = torch.full((B, Tq, H, 256), 2.0, dtype=o_dtype, device=cuda)
    S = rng.choice([0, 0, 3, 8])
    parts = (torch.empty(S, B, H, Tq, 256, device=cuda), torch.empty(S, B, H, Tq, device=cuda),
             torch.empty(S, B, H, Tq, device=cuda)) if S else (None, None, None)
    fa2.flash_attention(q_phys.permute(0, 2, 1, 3), k, v, o_phys.permute(0, 2, 1, 3), time, ph.to(cuda), ctx_window, 1,
                        *parts, stage=stage, scale=scale, sliding_window=sw, num_kv_splits=(S or None))
    o0 = torch.full((B, H, Tq, 256), 2.0)
    want = orc.flash_attention(case["q"], case["k"], case["v"], o0, case["time"], ph, ctx_window, 1, stage=stage,
                               scale=scale, sliding_window=sw)
    assert_close(o_phys.permute(0, 2, 1, 3), want, f"seed {seed}: H{H} G{G} B{B} Tq{Tq} T{T} cw{ctx_window} sw{sw} S{S}")


@pytest.mark.parametrize("seed", range(24))
def test_random_decode_paged(cuda, seed):
    rng = random.Random(3000 + seed)
    H, G = rng.choice([(8, 2), (4, 4), (16, 4), (6, 2), (16, 2), (5, 5)])
    B = rng.randint(1, 6)
    page = rng.choice([16, 16, 32, 64])
    lens = [rng.choice([1, 2, page - 1, page, page + 1, rng.randint(1, 3000)]) for _ in range(B)]
    dtype = rng.choice([torch.float16, torch.bfloat16])
    case = make_paged_case(4000 + seed, lens=lens, H=H, G=G, page_size=page, dtype=dtype)
    S = rng.choice([1, 2, 5, 16])
    sw = rng.choice([None, None, rng.randint(1, 500)])
    cw = rng.choice([case["max_len"], max(1, case["max_len"] // 2)])
    ph = _phase_vec(rng, B, 2)
    q, kp, vp, bt, time = (case[n].to(cuda) for n in ("q", "k_pool", "v_pool", "block_tables", "time"))
    o = torch.full((B, H, 1, 256), 2.0, dtype=dtype, device=cuda)
    po_dtype = rng.choice([torch.float32, torch.float16])
    po = torch.empty(S, B, H, 1, 256, dtype=po_dtype, device=cuda)
    pl, pm = torch.empty(S, B, H, 1, device=cuda), torch.empty(S, B, H, 1, device=cuda)
    fa2.flash_attention(q, kp, vp, o, time, ph.to(cuda), cw, 2, po, pl, pm, scale=1 / 16, sliding_window=sw,
                        block_tables=bt, page_size=page, num_kv_splits=S)
    want = orc.flash_attention(case["q"], case["k_pool"], case["v_pool"], torch.full((B, H, 1, 256), 2.0), case["time"], ph,
                               cw, 2, scale=1 / 16, sliding_window=sw, block_tables=case["block_tables"], page_size=page)
    tol = dict(abs_tol=4e-3, rel_tol=2e-2) if po_dtype == torch.float16 and S > 1 else {}
    assert_close(o, want, f"seed {seed}: H{H} G{G} lens{lens} page{page} S{S} sw{sw} cw{cw}", **tol)
