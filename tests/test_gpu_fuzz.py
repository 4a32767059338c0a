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
    # f16 partial accumulators (what the reference engine allocates, gemma4e.py:819-821) round
    # every split's un-normalised accumulator to 11 bits: relative 2^-11 per element, which after
    # the merge is at most 2^-11 x the largest |v| the slot attends to.  That bound is added to
    # the usual absolute term; the relative term stays.
    tol = {}
    if po_dtype == torch.float16 and S > 1:
        tol = dict(abs_tol=2e-3 + 2.0 ** -11 * float(case["v_pool"].float().abs().max()))
    assert_close(o, want, f"seed {seed}: H{H} G{G} lens{lens} page{page} S{S} sw{sw} cw{cw}", **tol)


@pytest.mark.parametrize("seed", range(16))
def test_random_prefill_paged(cuda, seed):
    from helpers import randn

    rng = random.Random(5000 + seed)
    H, G = rng.choice(HEADS)
    B = rng.randint(1, 3)
    page = rng.choice([16, 16, 32, 64])
    Tq = rng.choice([2, 31, 128, 150, 256, 333])
    times = [Tq + rng.choice([0, 1, page - 1, 77, 500, 1500]) for _ in range(B)]
    dtype = rng.choice([torch.float16, torch.bfloat16])
    case = make_paged_case(6000 + seed, lens=times, H=H, G=G, dtype=dtype, page_size=page)
    gen = torch.Generator().manual_seed(seed)
    q_phys = randn(gen, B, Tq, H, 256, dtype=dtype)
    # rows of the last page past each context hold NaN: they must never be multiplied in
    for b, n in enumerate(times):
        if n % page:
            last = int(case["block_tables"][b, (n - 1) // page])
            case["k_pool"][last, :, n % page:] = float("nan")
            case["v_pool"][last, :, n % page:] = float("nan")
    sw = rng.choice([None, None, rng.randint(1, 600)])
    cw = rng.choice([case["max_len"], case["max_len"], max(Tq, case["max_len"] // 2)])
    stage = rng.choice([fa2.STAGE_CAUSAL, fa2.STAGE_CAUSAL, fa2.STAGE_FULL])
    S = rng.choice([0, 0, 4])
    parts = (torch.empty(S, B, H, Tq, 256, device=cuda), torch.empty(S, B, H, Tq, device=cuda),
             torch.empty(S, B, H, Tq, device=cuda)) if S else (None, None, None)
    o_phys = torch.zeros(B, Tq, H, 256, dtype=dtype, device=cuda)
    fa2.flash_attention(q_phys.to(cuda).permute(0, 2, 1, 3), case["k_pool"].to(cuda), case["v_pool"].to(cuda),
                        o_phys.permute(0, 2, 1, 3), case["time"].to(cuda), None, cw, 1, *parts, stage=stage, scale=1 / 16,
                        sliding_window=sw, block_tables=case["block_tables"].to(cuda), page_size=page,
                        num_kv_splits=(S or None))
    kp = torch.nan_to_num(case["k_pool"].float(), nan=0.0)
    vp = torch.nan_to_num(case["v_pool"].float(), nan=0.0)
    want = orc.flash_attention(q_phys.permute(0, 2, 1, 3), kp, vp, torch.zeros(B, H, Tq, 256), case["time"], None, cw, 1,
                               stage=stage, scale=1 / 16, sliding_window=sw, block_tables=case["block_tables"], page_size=page)
    assert_close(o_phys.permute(0, 2, 1, 3), want, f"seed {seed}: H{H} G{G} times{times} Tq{Tq} page{page} sw{sw} cw{cw} S{S}")


@pytest.mark.parametrize("seed", range(12))
def test_random_rope_append(cuda, seed):
    from g4b_b200.kernels.rope import rope_norm_append
    from helpers import randn

    rng = random.Random(7000 + seed)
    H, G = rng.choice(HEADS)
    D = rng.choice([64, 128, 256, 256, 512])
    B, Tq = rng.randint(1, 3), rng.choice([1, 3, 40, 700])
    in_dtype = rng.choice([torch.float32, torch.float32, torch.bfloat16, torch.float16])
    c_dtype = rng.choice([torch.bfloat16, torch.float16, torch.float32])
    paged = rng.random() < 0.5
    gen = torch.Generator().manual_seed(seed)
    q, k, v = (randn(gen, B, Tq, h, D, dtype=in_dtype).permute(0, 2, 1, 3) for h in (H, G, G))
    qw, kw = 1 + 0.1 * randn(gen, D), 1 + 0.1 * randn(gen, D)
    freqs = 1.0 / (10000.0 ** (torch.arange(0, D, 2) / D))
    before = [rng.randint(0, 90) for _ in range(B)]
    off = torch.tensor(before, dtype=rng.choice([torch.int32, torch.int64]))
    ph = _phase_vec(rng, B, 1)
    if paged:
        page = rng.choice([16, 32])
        pages_per = [(b + Tq + page - 1) // page for b in before]
        n_pages = sum(pages_per) + 2
        perm = torch.randperm(n_pages, generator=gen).to(torch.int32)
        bt = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
        at = 0
        for b, n in enumerate(pages_per):
            bt[b, :n] = perm[at:at + n]
            at += n
        kc0, vc0 = randn(gen, n_pages, G, page, D, dtype=c_dtype), randn(gen, n_pages, G, page, D, dtype=c_dtype)
        extra = dict(block_tables=bt, page_size=page)
    else:
        T = Tq + rng.randint(0, 50)
        kc0, vc0 = randn(gen, B, G, T, D, dtype=c_dtype), randn(gen, B, G, T, D, dtype=c_dtype)
        extra = {}
    norm_qk, norm_v, rotate = rng.random() < 0.8, rng.random() < 0.7, rng.random() < 0.85
    want_q, _, want_kc, want_vc = orc.rope_norm_append(q, k, v, freqs if rotate else None, off, kc0, vc0, 1e-6,
                                                       q_rmsnorm_w=qw, k_rmsnorm_w=kw, norm_qk=norm_qk, norm_v=norm_v,
                                                       user_phase=ph, phase=1, **extra)
    kc, vc = kc0.to(cuda), vc0.to(cuda)
    q_out = torch.zeros(B, H, Tq, D, dtype=c_dtype, device=cuda)
    dev_extra = {key: (val.to(cuda) if torch.is_tensor(val) else val) for key, val in extra.items()}
    rope_norm_append(q.to(cuda), k.to(cuda), v.to(cuda), freqs.to(cuda) if rotate else None, off.to(cuda), kc, vc, 1e-6,
                     q_out=q_out, q_rmsnorm_w=qw.to(cuda), k_rmsnorm_w=kw.to(cuda), norm_qk=norm_qk, norm_v=norm_v,
                     user_phase=ph.to(cuda), phase=1, **dev_extra)
    tol = {torch.float32: 3e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[c_dtype]
    what = f"seed {seed}: H{H} G{G} D{D} B{B} Tq{Tq} {in_dtype}->{c_dtype} paged={paged}"
    assert torch.allclose(q_out.float().cpu(), want_q, atol=tol, rtol=tol), what
    assert torch.allclose(kc.float().cpu(), want_kc.float(), atol=tol, rtol=tol), what
    assert torch.allclose(vc.float().cpu(), want_vc.float(), atol=tol, rtol=tol), what


@pytest.mark.parametrize("seed", range(16))
def test_random_kv_append(cuda, seed):
    """add_kv_to_cache over head dims off the 8-element grid, rows that start off a 16-byte
    boundary (the element-wise path), token counts off the four-row grouping, rings written
    completely (Tq = T) and wrapped, pages, slots off phase, both offset types."""
    from g4b_b200.kernels.add_kv_to_cache import add_kv_to_cache
    from helpers import randn

    rng = random.Random(9000 + seed)
    B, G = rng.randint(1, 4), rng.choice([1, 2, 4, 5])
    D = rng.choice([256, 256, 64, 40, 36, 30, 512, 264])
    Tq = rng.choice([1, 2, 3, 4, 5, 7, 8, 31, 64, 130])
    x_dtype = rng.choice([torch.float32, torch.float16, torch.bfloat16])
    c_dtype = rng.choice([x_dtype, torch.float16, torch.bfloat16, torch.float32])
    norm = rng.random() < 0.5
    paged = rng.random() < 0.4
    shift = rng.choice([0, 0, 1, 3])               # elements the rows start past an aligned address
    gen = torch.Generator().manual_seed(seed)
    x_phys = randn(gen, B, Tq, G, D + shift, dtype=x_dtype)
    x = x_phys[..., shift:].permute(0, 2, 1, 3)
    rsos = (x.float() ** 2).sum(-1) if norm else None
    phase = _phase_vec(rng, B, 1) if rng.random() < 0.5 else None
    off_dtype = rng.choice([torch.int32, torch.int64])
    if paged:
        page = rng.choice([16, 32])
        per_seq = (Tq + 50 + page - 1) // page + 1
        n_pages = B * per_seq + 3
        cache = randn(gen, n_pages, G, page, D, dtype=c_dtype)
        bt = torch.randperm(n_pages, generator=gen)[: B * per_seq].to(torch.int32).view(B, per_seq)
        off = torch.tensor([rng.randint(0, 50) for _ in range(B)], dtype=off_dtype)
        kw = dict(block_tables=bt, page_size=page)
        kw_d = dict(block_tables=bt.to(cuda), page_size=page)
    else:
        T = Tq + rng.choice([0, 0, 1, 9, 100])
        cache = randn(gen, B, G, T, D, dtype=c_dtype)
        off = torch.tensor([rng.randint(0, 3 * T) for _ in range(B)], dtype=off_dtype)
        kw, kw_d = {}, {}
    want = orc.add_kv_to_cache(x, cache, off, 1e-6, rsos, phase, 1, **kw)
    cache_d = cache.to(cuda)
    xd = x_phys.to(cuda)[..., shift:].permute(0, 2, 1, 3)
    add_kv_to_cache(xd, cache_d, off.to(cuda), 1e-6, None if rsos is None else rsos.to(cuda),
                    None if phase is None else phase.to(cuda), 1, **kw_d)
    what = f"seed {seed}: B{B} G{G} D{D} Tq{Tq} {x_dtype}->{c_dtype} norm{norm} paged{paged} shift{shift}"
    if norm:
        tol = {torch.float32: 2e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[c_dtype]
        assert torch.allclose(cache_d.cpu().float(), want.float(), rtol=tol, atol=tol), what
    else:
        assert torch.equal(cache_d.cpu().view(torch.uint8), want.view(torch.uint8)), what
