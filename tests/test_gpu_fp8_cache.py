"""The 8-bit (e4m3) paged KV cache: the quantising append bit-exact against the CPU restatement
of the quantiser, and Tq == 1 attention over the 8-bit pools against the oracle's attention on
the de-quantised values, at the tolerance of every other parity test."""
import random

import pytest
import torch

from g4b_b200.kernels import fa2
from g4b_b200.kernels.add_kv_to_cache import add_kv_to_cache_fp8
from helpers import assert_close, orc, randn

pytestmark = pytest.mark.gpu


def _tables(gen, lens, page, extra=2):
    pages_per = [(n + page - 1) // page for n in lens]
    num_pages = sum(pages_per) + extra
    perm = torch.randperm(num_pages, generator=gen)
    bt = torch.full((len(lens), max(pages_per)), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages_per):
        bt[b, :n] = perm[at:at + n].to(torch.int32)
        at += n
    return bt, num_pages


@pytest.mark.parametrize("in_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,page", [(256, 16), (128, 32), (512, 16)])
def test_append_quantises_bit_exactly_however_the_rows_are_chunked(cuda, in_dtype, D, page):
    gen = torch.Generator().manual_seed(D + page)
    B, G = 3, 2
    lens = [3 * page + 5, page, 2 * page + 1]
    bt, num_pages = _tables(gen, lens, page)
    x = [randn(gen, 1, G, n, D, dtype=in_dtype) * (0.2 + b) for b, n in enumerate(lens)]
    # oracle: every sequence in one go
    want_pool = torch.zeros(num_pages, G, page, D, dtype=torch.uint8)
    want_sc = torch.zeros(num_pages, G)
    for b, n in enumerate(lens):
        want_pool, want_sc = orc.add_kv_to_cache_fp8(x[b], want_pool, want_sc, torch.tensor([0]), 1e-6,
                                                     block_tables=bt[b:b + 1], page_size=page)
    # GPU: a first chunk of 1.5 pages for all slots at once (padded batch), then the rest row by row
    pool = torch.zeros(num_pages, G, page, D, dtype=torch.uint8, device=cuda)
    sc = torch.zeros(num_pages, G, device=cuda)
    btd = bt.to(cuda)
    first = page + page // 2
    for b, n in enumerate(lens):
        c = min(first, n)
        add_kv_to_cache_fp8(x[b][:, :, :c].to(cuda), pool, sc, torch.tensor([0], dtype=torch.int32, device=cuda), 1e-6,
                            block_tables=btd[b:b + 1], page_size=page)
        for t in range(c, n, 7):
            e = min(n, t + 7)
            add_kv_to_cache_fp8(x[b][:, :, t:e].to(cuda), pool, sc, torch.tensor([t], dtype=torch.int64, device=cuda), 1e-6,
                                block_tables=btd[b:b + 1], page_size=page)
    assert torch.equal(sc.cpu(), want_sc), "page scales differ"
    assert torch.equal(pool.cpu(), want_pool), "stored bytes differ"


def test_append_with_v_norm_and_phase_gate(cuda):
    gen = torch.Generator().manual_seed(5)
    B, G, D, page, Tq = 2, 2, 256, 16, 16
    bt, num_pages = _tables(gen, [Tq, Tq], page)
    x = randn(gen, B, G, Tq, D)
    rsos = (x ** 2).sum(-1)
    phase = torch.tensor([1, 2], dtype=torch.uint8)
    off = torch.zeros(B, dtype=torch.int32)
    want_pool, want_sc = orc.add_kv_to_cache_fp8(x, torch.zeros(num_pages, G, page, D, dtype=torch.uint8),
                                                 torch.zeros(num_pages, G), off, 1e-6, rsos, phase, 2, block_tables=bt,
                                                 page_size=page)
    pool = torch.zeros(num_pages, G, page, D, dtype=torch.uint8, device=cuda)
    sc = torch.zeros(num_pages, G, device=cuda)
    add_kv_to_cache_fp8(x.to(cuda), pool, sc, off.to(cuda), 1e-6, rsos.to(cuda), phase.to(cuda), 2, block_tables=bt.to(cuda),
                        page_size=page)
    # the norm's rsqrt is an approximation on both sides: scales agree to a few ulp, values to one e4m3 step
    assert torch.allclose(sc.cpu(), want_sc, rtol=1e-6, atol=0)
    got, want = orc.dequantise_fp8_pool(pool.cpu(), sc.cpu()), orc.dequantise_fp8_pool(want_pool, want_sc)
    assert bool(((got - want).abs() <= 0.125 * want.abs() + 1e-6).all())
    assert float(((got != want).float().mean())) < 1e-3
    assert float(pool.cpu()[bt[0, 0].long()].float().abs().sum()) == 0, "the off-phase slot's page was written"


@pytest.mark.parametrize("seed", range(10))
def test_attention_over_fp8_pools(cuda, seed):
    rng = random.Random(9100 + seed)
    D = rng.choice([128, 256, 256, 512])
    H, G = rng.choice([(8, 2), (4, 4), (16, 4), (16, 2)])
    page = rng.choice([16, 32])
    B = rng.randint(1, 4)
    lens = [rng.choice([1, page, page + 1, rng.randint(1, 2500)]) for _ in range(B)]
    gen = torch.Generator().manual_seed(seed)
    bt, num_pages = _tables(gen, lens, page)
    # pools filled by the quantising append (so scales and bytes are what a serving loop would hold)
    kp = torch.zeros(num_pages, G, page, D, dtype=torch.uint8)
    vp = torch.zeros_like(kp)
    ks, vs = torch.zeros(num_pages, G), torch.zeros(num_pages, G)
    for b, n in enumerate(lens):
        kx, vx = randn(gen, 1, G, n, D), randn(gen, 1, G, n, D)
        kp, ks = orc.add_kv_to_cache_fp8(kx, kp, ks, torch.tensor([0]), 1e-6, block_tables=bt[b:b + 1], page_size=page)
        vp, vs = orc.add_kv_to_cache_fp8(vx, vp, vs, torch.tensor([0]), 1e-6, block_tables=bt[b:b + 1], page_size=page)
    # unused rows of the last pages hold NaN bytes: they must never be multiplied in
    for b, n in enumerate(lens):
        if n % page:
            last = int(bt[b, (n - 1) // page])
            kp[last, :, n % page:] = 0x7f
            vp[last, :, n % page:] = 0xff
    q_dtype = rng.choice([torch.float16, torch.bfloat16, torch.float32])
    q = randn(gen, B, H, 1, D, dtype=q_dtype)
    time = torch.tensor(lens, dtype=torch.int32)
    cw = bt.shape[1] * page
    sw = rng.choice([None, None, rng.randint(1, 300)])
    S = rng.choice([1, 3, 8])
    ph = torch.tensor([rng.choice([2, 2, 0]) for _ in range(B)], dtype=torch.uint8)
    o0 = torch.full((B, H, 1, D), 1.5)
    kd, vd = orc.dequantise_fp8_pool(kp, ks), orc.dequantise_fp8_pool(vp, vs)
    kd, vd = torch.nan_to_num(kd), torch.nan_to_num(vd)           # only rows past the contexts
    # q reaches the tensor cores as f16
    want = orc.flash_attention(q.to(torch.float16), kd, vd, o0, time, ph, cw, 2, scale=1 / 16, sliding_window=sw,
                               block_tables=bt, page_size=page)
    o = o0.to(torch.float16).to(cuda)
    parts = ()
    if S > 1:
        parts = (torch.empty(S, B, H, 1, D, device=cuda), torch.empty(S, B, H, 1, device=cuda), torch.empty(S, B, H, 1, device=cuda))
    fa2.flash_attention_fp8(q.to(cuda), kp.to(cuda), vp.to(cuda), ks.to(cuda), vs.to(cuda), o, time.to(cuda), ph.to(cuda), cw,
                            fa2.PHASE_DECODE, *parts, block_tables=bt.to(cuda), page_size=page, scale=1 / 16,
                            sliding_window=sw, num_kv_splits=S if S > 1 else None)
    assert_close(o, want, f"seed {seed}: D{D} H{H} G{G} page{page} lens{lens} S{S} sw{sw}")


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D,page", [(256, 16), (128, 32), (512, 16)])
def test_dequantised_pool_is_bit_exact(cuda, out_dtype, D, page):
    """Every byte value (NaN codes apart) under a spread of scales: out = round(e4m3 x scale),
    whole pool and restricted to the pages of the slots in phase."""
    from g4b_b200.kernels.add_kv_to_cache import dequantise_fp8_pool

    gen = torch.Generator().manual_seed(D + page)
    G, lens = 2, [3 * page + 5, page, 1, 2 * page]
    bt, num_pages = _tables(gen, lens, page, extra=3)
    pool = torch.randint(0, 256, (num_pages, G, page, D), generator=gen, dtype=torch.int16).to(torch.uint8)
    pool[(pool & 0x7f) == 0x7f] = 0x3c                                   # no NaN codes
    sc = torch.rand(num_pages, G, generator=gen) * torch.tensor([1e-3, 1.0, 37.0])[torch.randint(0, 3, (num_pages, G), generator=gen)]
    want = orc.dequantise_fp8_pool(pool, sc).to(out_dtype)
    out = torch.full((num_pages, G, page, D), 9.0, dtype=out_dtype, device=cuda)
    dequantise_fp8_pool(pool.to(cuda), sc.to(cuda), out, page_size=page)
    assert torch.equal(out.cpu(), want)
    # restricted: slots 0 and 3 are in phase 1, slot 1 is not; slot 2 holds one token
    out.fill_(9.0)
    time = torch.tensor(lens, dtype=torch.int32)
    ph = torch.tensor([1, 0, 1, 1], dtype=torch.uint8)
    dequantise_fp8_pool(pool.to(cuda), sc.to(cuda), out, block_tables=bt.to(cuda), time_dim_sizes=time.to(cuda),
                        user_phase=ph.to(cuda), phase=1, page_size=page)
    live = torch.zeros(num_pages, dtype=torch.bool)
    for b, n in enumerate(lens):
        if ph[b] == 1:
            live[bt[b, :(n + page - 1) // page].long()] = True
    got = out.cpu()
    assert torch.equal(got[live], want[live])
    assert bool((got[~live] == 9.0).all()), "pages outside the request were written"


def test_prefill_chunk_over_an_8_bit_context(cuda):
    """A chunk of 96 new tokens attends to a context that lives in e4m3 pages: append (quantise)
    the chunk, de-quantise the slots' pages into a 16-bit scratch pool, run the prefill kernel
    over it with the same block tables; against the oracle's attention on the de-quantised values."""
    from g4b_b200.kernels.add_kv_to_cache import dequantise_fp8_pool

    gen = torch.Generator().manual_seed(77)
    B, H, G, D, page, Tq = 2, 8, 2, 256, 16, 96
    ctx = [700, 333]                                                       # tokens already cached
    lens = [c + Tq for c in ctx]
    bt, num_pages = _tables(gen, lens, page)
    kp = torch.zeros(num_pages, G, page, D, dtype=torch.uint8)
    vp = torch.zeros_like(kp)
    ks, vs = torch.zeros(num_pages, G), torch.zeros(num_pages, G)
    for b, n in enumerate(ctx):
        kp, ks = orc.add_kv_to_cache_fp8(randn(gen, 1, G, n, D), kp, ks, torch.tensor([0]), 1e-6, block_tables=bt[b:b + 1], page_size=page)
        vp, vs = orc.add_kv_to_cache_fp8(randn(gen, 1, G, n, D), vp, vs, torch.tensor([0]), 1e-6, block_tables=bt[b:b + 1], page_size=page)
    k_new, v_new = randn(gen, B, G, Tq, D), randn(gen, B, G, Tq, D)
    q = randn(gen, B, H, Tq, D, dtype=torch.bfloat16)
    off = torch.tensor(ctx, dtype=torch.int32)
    time = torch.tensor(lens, dtype=torch.int32)
    # oracle: quantise the chunk, de-quantise everything, attend
    wkp, wks = orc.add_kv_to_cache_fp8(k_new, kp.clone(), ks.clone(), off, 1e-6, block_tables=bt, page_size=page)
    wvp, wvs = orc.add_kv_to_cache_fp8(v_new, vp.clone(), vs.clone(), off, 1e-6, block_tables=bt, page_size=page)
    kd = orc.dequantise_fp8_pool(wkp, wks).to(torch.bfloat16).float()
    vd = orc.dequantise_fp8_pool(wvp, wvs).to(torch.bfloat16).float()
    cw = bt.shape[1] * page
    want = orc.flash_attention(q, kd, vd, torch.zeros(B, H, Tq, D), time, None, cw, 1, scale=1 / 16, block_tables=bt, page_size=page)
    # GPU
    dkp, dvp, dks, dvs, dbt = kp.to(cuda), vp.to(cuda), ks.to(cuda), vs.to(cuda), bt.to(cuda)
    add_kv_to_cache_fp8(k_new.to(cuda), dkp, dks, off.to(cuda), 1e-6, block_tables=dbt, page_size=page)
    add_kv_to_cache_fp8(v_new.to(cuda), dvp, dvs, off.to(cuda), 1e-6, block_tables=dbt, page_size=page)
    assert torch.equal(dkp.cpu(), wkp) and torch.equal(dvp.cpu(), wvp)
    k16 = torch.zeros(num_pages, G, page, D, dtype=torch.bfloat16, device=cuda)
    v16 = torch.zeros_like(k16)
    dequantise_fp8_pool(dkp, dks, k16, block_tables=dbt, time_dim_sizes=time.to(cuda), page_size=page)
    dequantise_fp8_pool(dvp, dvs, v16, block_tables=dbt, time_dim_sizes=time.to(cuda), page_size=page)
    o = torch.zeros(B, H, Tq, D, dtype=torch.bfloat16, device=cuda)
    fa2.flash_attention(q.to(cuda), k16, v16, o, time.to(cuda), None, cw, fa2.PHASE_PREFILL, scale=1 / 16,
                        block_tables=dbt, page_size=page)
    assert_close(o, want, "prefill chunk over an 8-bit context")


def test_serving_loop_over_8_bit_pages(cuda):
    """Two requests through chunked prefill and decode with nothing but 8-bit pages behind them:
    every chunk is quantised into the pages, the slot's pages are converted into a 16-bit scratch
    pool and the prefill kernel attends over it; every decode step appends one row per slot and
    attends over the bytes.  After every step the pools equal the CPU quantiser's bit for bit and
    the attention output equals the oracle's attention over the de-quantised values."""
    from g4b_b200.kernels.add_kv_to_cache import dequantise_fp8_pool

    gen = torch.Generator().manual_seed(2024)
    B, H, G, D, page, CHUNK, n_decode = 2, 8, 2, 256, 16, 32, 5
    prompts = [70, 45]
    bt, num_pages = _tables(gen, [n + n_decode for n in prompts], page)
    cw = bt.shape[1] * page
    # CPU twins of the pools, advanced by the oracle's quantiser
    wk, wv = torch.zeros(num_pages, G, page, D, dtype=torch.uint8), torch.zeros(num_pages, G, page, D, dtype=torch.uint8)
    wks, wvs = torch.zeros(num_pages, G), torch.zeros(num_pages, G)
    dk, dv, dks, dvs = wk.to(cuda), wv.to(cuda), wks.to(cuda), wvs.to(cuda)
    k16 = torch.zeros(num_pages, G, page, D, dtype=torch.bfloat16, device=cuda)
    v16 = torch.zeros_like(k16)
    dbt = bt.to(cuda)
    for b, n in enumerate(prompts):                      # ---- chunked prefill, one slot at a time
        for s in range(0, n, CHUNK):
            e = min(n, s + CHUNK)
            kx, vx = randn(gen, 1, G, e - s, D), randn(gen, 1, G, e - s, D)
            q = randn(gen, 1, H, e - s, D, dtype=torch.bfloat16)
            off, time = torch.tensor([s], dtype=torch.int32), torch.tensor([e], dtype=torch.int32)
            wk, wks = orc.add_kv_to_cache_fp8(kx, wk, wks, off, 1e-6, block_tables=bt[b:b + 1], page_size=page)
            wv, wvs = orc.add_kv_to_cache_fp8(vx, wv, wvs, off, 1e-6, block_tables=bt[b:b + 1], page_size=page)
            add_kv_to_cache_fp8(kx.to(cuda), dk, dks, off.to(cuda), 1e-6, block_tables=dbt[b:b + 1], page_size=page)
            add_kv_to_cache_fp8(vx.to(cuda), dv, dvs, off.to(cuda), 1e-6, block_tables=dbt[b:b + 1], page_size=page)
            assert torch.equal(dk.cpu(), wk) and torch.equal(dv.cpu(), wv), f"slot {b} chunk at {s}: bytes differ"
            dequantise_fp8_pool(dk, dks, k16, block_tables=dbt[b:b + 1], time_dim_sizes=time.to(cuda), page_size=page)
            dequantise_fp8_pool(dv, dvs, v16, block_tables=dbt[b:b + 1], time_dim_sizes=time.to(cuda), page_size=page)
            o = torch.zeros(1, H, e - s, D, dtype=torch.bfloat16, device=cuda)
            fa2.flash_attention(q.to(cuda), k16, v16, o, time.to(cuda), None, cw, fa2.PHASE_PREFILL, scale=1 / 16,
                                block_tables=dbt[b:b + 1], page_size=page)
            kd = orc.dequantise_fp8_pool(wk, wks).to(torch.bfloat16).float()
            vd = orc.dequantise_fp8_pool(wv, wvs).to(torch.bfloat16).float()
            want = orc.flash_attention(q, kd, vd, torch.zeros(1, H, e - s, D), time, None, cw, 1, scale=1 / 16,
                                       block_tables=bt[b:b + 1], page_size=page)
            assert_close(o, want, f"slot {b} prefill chunk [{s}, {e})")
    pos = torch.tensor(prompts, dtype=torch.int32)       # ---- decode, both slots per step
    parts = (torch.empty(3, B, H, 1, D, device=cuda), torch.empty(3, B, H, 1, device=cuda), torch.empty(3, B, H, 1, device=cuda))
    for step in range(n_decode):
        kx, vx = randn(gen, B, G, 1, D), randn(gen, B, G, 1, D)
        q = randn(gen, B, H, 1, D, dtype=torch.float16)
        wk, wks = orc.add_kv_to_cache_fp8(kx, wk, wks, pos, 1e-6, block_tables=bt, page_size=page)
        wv, wvs = orc.add_kv_to_cache_fp8(vx, wv, wvs, pos, 1e-6, block_tables=bt, page_size=page)
        add_kv_to_cache_fp8(kx.to(cuda), dk, dks, pos.to(cuda), 1e-6, block_tables=dbt, page_size=page)
        add_kv_to_cache_fp8(vx.to(cuda), dv, dvs, pos.to(cuda), 1e-6, block_tables=dbt, page_size=page)
        assert torch.equal(dk.cpu(), wk) and torch.equal(dv.cpu(), wv) and torch.equal(dks.cpu(), wks), f"decode step {step}: pools differ"
        time = pos + 1
        o = torch.zeros(B, H, 1, D, dtype=torch.float16, device=cuda)
        fa2.flash_attention_fp8(q.to(cuda), dk, dv, dks, dvs, o, time.to(cuda), None, cw, fa2.PHASE_DECODE, *parts,
                                block_tables=dbt, page_size=page, scale=1 / 16, num_kv_splits=3)
        want = orc.flash_attention(q, orc.dequantise_fp8_pool(wk, wks), orc.dequantise_fp8_pool(wv, wvs),
                                   torch.zeros(B, H, 1, D), time, None, cw, 2, scale=1 / 16, block_tables=bt, page_size=page)
        assert_close(o, want, f"decode step {step}")
        pos = pos + 1
