"""g4b_decode_step: append + decode attention, then the merge of the splits (or, with peers, the
merge and the exchange inside the attention launch), against the oracle; and the TMA-fed decode
kernel under it at head dims 128 / 512, at the ring's wrap, with ragged edges and with splits
that see no key.

The exchange is tested on one GPU with the test playing the peers: their words are in this
rank's buffer before the launch, so no kernel waits for another kernel."""
import random

import pytest
import torch

from g4b_b200 import _cabi
from g4b_b200.dist import PartialExchange
from g4b_b200.kernels import fa2
from helpers import assert_close, make_paged_case, make_ring_case, orc, randn

pytestmark = pytest.mark.gpu


def _workspace(S, B, H, D, cuda, packed=False):
    if packed:   # one [S,B,H,1,D+2] buffer holding all three, rows on 8-byte boundaries only
        buf = torch.empty(S, B, H, 1, D + 2, device=cuda)
        return buf[..., :D], buf[..., D], buf[..., D + 1]
    return torch.empty(S, B, H, 1, D, device=cuda), torch.empty(S, B, H, 1, device=cuda), torch.empty(S, B, H, 1, device=cuda)


@pytest.mark.parametrize("D", [128, 256, 512])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_decode_kernel_head_dims_paged_and_ring(cuda, D, dtype):
    """The plain entry points (flash_attention with and without splits) at every head dim."""
    case = make_paged_case(300 + D, lens=[1, 15, 16, 17, 700, 2049], H=8, G=2, D=D, dtype=dtype)
    q, kp, vp, bt, time = (case[n].to(cuda) for n in ("q", "k_pool", "v_pool", "block_tables", "time"))
    want = orc.flash_attention(case["q"], case["k_pool"], case["v_pool"], torch.zeros(6, 8, 1, D), case["time"], None,
                               case["max_len"], 2, scale=1 / 16, block_tables=case["block_tables"], page_size=16)
    for S in (1, 5):
        o = torch.zeros(6, 8, 1, D, dtype=dtype, device=cuda)
        parts = _workspace(S, 6, 8, D, cuda) if S > 1 else ()
        fa2.flash_attention(q, kp, vp, o, time, None, case["max_len"], fa2.PHASE_DECODE, *parts, scale=1 / 16,
                            block_tables=bt, page_size=16, num_kv_splits=S if S > 1 else None)
        assert_close(o, want, f"paged D{D} S{S}")
    ring = make_ring_case(310 + D, B=3, H=4, G=2, Tq=1, T=200, D=D, dtype=dtype, times=[200, 217, 90], ctx_window=200)
    o = torch.zeros(3, 4, 1, D, dtype=dtype, device=cuda)
    fa2.flash_attention(ring["q"].to(cuda), ring["k"].to(cuda), ring["v"].to(cuda), o, ring["time"].to(cuda), None, 200,
                        fa2.PHASE_DECODE, scale=1 / 16)
    want = orc.flash_attention(ring["q"], ring["k"], ring["v"], torch.zeros(3, 4, 1, D), ring["time"], None, 200, 2,
                               scale=1 / 16)
    assert_close(o, want, f"ring D{D}")


@pytest.mark.parametrize("seed", range(12))
def test_ring_wrap_positions(cuda, seed):
    """The ring's wrap at every offset inside a 16-key block, window edges that are not block
    aligned, NaN in rows the window does not expose."""
    rng = random.Random(7100 + seed)
    B, H, G, D = 3, 8, 2, 256
    T = rng.choice([16, 17, 31, 64, 100, 333])
    cw = rng.randint(max(1, T - 20), T)
    times = [rng.choice([cw + rng.randint(0, 3 * T), rng.randint(1, cw), cw]) for _ in range(B)]
    dtype = rng.choice([torch.float16, torch.bfloat16])
    case = make_ring_case(7200 + seed, B=B, H=H, G=G, Tq=1, T=T, D=D, dtype=dtype, times=times, ctx_window=cw)
    sw = rng.choice([None, rng.randint(1, cw)])
    k, v = case["k"].clone(), case["v"].clone()
    for b, t in enumerate(times):          # rows outside the exposed window may hold anything
        window = min(t, cw)
        start = max(t - cw, 0) % T
        dead = [r for r in range(T) if (r - start) % T >= window]
        if dead:
            k[b, :, dead], v[b, :, dead] = float("nan"), float("nan")
    S = rng.choice([1, 2, 3])
    o = torch.zeros(B, H, 1, D, dtype=dtype, device=cuda)
    parts = _workspace(S, B, H, D, cuda) if S > 1 else ()
    fa2.flash_attention(case["q"].to(cuda), k.to(cuda), v.to(cuda), o, case["time"].to(cuda), None, cw, fa2.PHASE_DECODE,
                        *parts, scale=1 / 16, sliding_window=sw, num_kv_splits=S if S > 1 else None)
    want = orc.flash_attention(case["q"], case["k"], case["v"], torch.zeros(B, H, 1, D), case["time"], None, cw, 2,
                               scale=1 / 16, sliding_window=sw)
    assert_close(o, want, f"T{T} cw{cw} times{times} sw{sw} S{S}")


@pytest.mark.parametrize("S", [1, 2, 8, 9, 16, 40, 148])
@pytest.mark.parametrize("packed", [False, True])
def test_decode_step_paged_with_append(cuda, S, packed):
    """Append + attention + merge for a range of split counts; called three times in a row (the
    workspace holds the previous call's partials).  Slot 2 is off phase."""
    lens = [3000, 17, 555, 1, 4096]
    B, H, G, D = len(lens), 8, 2, 256
    case = make_paged_case(400 + S, lens=lens, H=H, G=G, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(S)
    k_new, v_new = randn(gen, B, G, 1, D, dtype=torch.bfloat16), randn(gen, B, G, 1, D, dtype=torch.bfloat16)
    phase = torch.tensor([2, 2, 1, 2, 2], dtype=torch.uint8)
    off = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    want_k = orc.add_kv_to_cache(k_new, case["k_pool"], off, 1e-6, None, phase, 2, block_tables=case["block_tables"], page_size=16)
    want_v = orc.add_kv_to_cache(v_new, case["v_pool"], off, 1e-6, None, phase, 2, block_tables=case["block_tables"], page_size=16)
    want = orc.flash_attention(case["q"], want_k, want_v, torch.full((B, H, 1, D), 7.0), case["time"], phase,
                               case["max_len"], 2, scale=1 / 16, block_tables=case["block_tables"], page_size=16)
    q, bt, time = case["q"].to(cuda), case["block_tables"].to(cuda), case["time"].to(cuda)
    po, pl, pm = _workspace(S, B, H, D, cuda, packed)
    for rep in range(3):
        kp, vp = case["k_pool"].to(cuda), case["v_pool"].to(cuda)
        o = torch.full((B, H, 1, D), 7.0, dtype=torch.bfloat16, device=cuda)
        fa2.decode_step(q, kp, vp, o, time, phase.to(cuda), case["max_len"], fa2.PHASE_DECODE, po, pl, pm,
                        k_new=k_new.to(cuda), v_new=v_new.to(cuda), num_kv_splits=S, scale=1 / 16, block_tables=bt,
                        page_size=16)
        assert_close(o, want, f"decode step S{S} rep{rep}")
        assert torch.equal(kp.cpu(), want_k) and torch.equal(vp.cpu(), want_v), "appended rows differ"
    assert _cabi.device_status() == 0


@pytest.mark.parametrize("seed", range(10))
def test_decode_step_random(cuda, seed):
    """Seeded sweep: rings and pages, head dims, dtypes, f32 q, group sizes, windows, with and
    without the append, against the oracle."""
    rng = random.Random(8100 + seed)
    D = rng.choice([128, 256, 256, 512])
    H, G = rng.choice([(8, 2), (4, 4), (16, 4), (6, 2), (16, 2)])
    B = rng.randint(1, 4)
    dtype = rng.choice([torch.float16, torch.bfloat16])
    S = rng.choice([1, 3, 8, 11, 24])
    paged = rng.random() < 0.5
    append = rng.random() < 0.6
    ph = torch.tensor([rng.choice([2, 2, 2, 0]) for _ in range(B)], dtype=torch.uint8)
    gen = torch.Generator().manual_seed(seed)
    k_new, v_new = randn(gen, B, G, 1, D, dtype=dtype), randn(gen, B, G, 1, D, dtype=dtype)
    o0 = torch.full((B, H, 1, D), -3.0)
    if paged:
        page = rng.choice([16, 32, 64])
        lens = [rng.choice([1, page, page + 1, rng.randint(1, 2500)]) for _ in range(B)]
        case = make_paged_case(8200 + seed, lens=lens, H=H, G=G, D=D, page_size=page, dtype=dtype)
        cw = rng.choice([case["max_len"], max(1, case["max_len"] // 2)])
        sw = rng.choice([None, rng.randint(1, 400)])
        kc, vc, extra = case["k_pool"], case["v_pool"], dict(block_tables=case["block_tables"], page_size=page)
        off = case["time"] - 1
    else:
        T = rng.choice([16, 50, 257, 1024])
        cw = rng.randint(max(1, T - 30), T)
        times = [rng.choice([cw, cw + rng.randint(1, 2 * T), rng.randint(1, cw)]) for _ in range(B)]
        case = make_ring_case(8300 + seed, B=B, H=H, G=G, Tq=1, T=T, D=D, dtype=dtype, times=times, ctx_window=cw)
        sw = rng.choice([None, rng.randint(1, cw)])
        kc, vc, extra = case["k"], case["v"], {}
        off = (case["time"] - 1) % T
    q = case["q"].float() if rng.random() < 0.3 else case["q"]
    want_k, want_v = kc, vc
    if append:
        want_k = orc.add_kv_to_cache(k_new, kc, off, 1e-6, None, ph, 2, **extra)
        want_v = orc.add_kv_to_cache(v_new, vc, off, 1e-6, None, ph, 2, **extra)
    want = orc.flash_attention(q, want_k, want_v, o0, case["time"], ph, cw, 2, scale=1 / 16, sliding_window=sw, **extra)
    kd, vd = kc.to(cuda), vc.to(cuda)
    o = o0.to(dtype).to(cuda)
    po, pl, pm = _workspace(S, B, H, D, cuda, packed=rng.random() < 0.5)
    dev_extra = {k: (v.to(cuda) if hasattr(v, "to") else v) for k, v in extra.items()}
    fa2.decode_step(q.to(cuda), kd, vd, o, case["time"].to(cuda), ph.to(cuda), cw, fa2.PHASE_DECODE, po, pl, pm,
                    k_new=k_new.to(cuda) if append else None, v_new=v_new.to(cuda) if append else None,
                    num_kv_splits=S, scale=1 / 16, sliding_window=sw, **dev_extra)
    assert_close(o, want, f"seed {seed}: D{D} H{H} G{G} B{B} S{S} paged{paged} append{append} sw{sw} cw{cw}")
    assert torch.equal(kd.cpu(), want_k) and torch.equal(vd.cpu(), want_v), "cache after the step differs"


def test_decode_step_matches_two_launch_path_at_benchmark_size(cuda):
    """One sequence of 131072 tokens (shuffled pages): the one-launch step, the decode + combine
    path and the oracle agree; size-independent property: the result does not depend on the
    split count."""
    L, H, G, D = 131072, 8, 2, 256
    gen = torch.Generator(device=cuda).manual_seed(5)
    n_pages = L // 16
    kp = torch.randn(n_pages, G, 16, D, generator=gen, device=cuda).to(torch.bfloat16)
    vp = torch.randn(n_pages, G, 16, D, generator=gen, device=cuda).to(torch.bfloat16)
    bt = torch.randperm(n_pages, generator=torch.Generator().manual_seed(6)).to(torch.int32)[None].to(cuda)
    q = torch.randn(1, H, 1, D, generator=gen, device=cuda).to(torch.bfloat16)
    time = torch.tensor([L], dtype=torch.int32, device=cuda)
    k = kp[bt[0].long()].float().cpu().permute(1, 0, 2, 3).reshape(G, L, D)
    v = vp[bt[0].long()].float().cpu().permute(1, 0, 2, 3).reshape(G, L, D)
    want = orc.attention_core(q[0].float().cpu(), k, v, scale=1 / 16)[None]
    outs = []
    for S in (16, 74, 148):
        po, pl, pm = _workspace(S, 1, H, D, cuda, packed=True)
        o = torch.zeros(1, H, 1, D, dtype=torch.bfloat16, device=cuda)
        fa2.decode_step(q, kp, vp, o, time, None, L, fa2.PHASE_DECODE, po, pl, pm, num_kv_splits=S, scale=1 / 16,
                        block_tables=bt, page_size=16)
        assert_close(o, want, f"decode step, {S} splits")
        o2 = torch.zeros_like(o)
        fa2.flash_attention(q, kp, vp, o2, time, None, L, fa2.PHASE_DECODE, po, pl, pm, num_kv_splits=S, scale=1 / 16,
                            block_tables=bt, page_size=16)
        assert_close(o2, want, f"two launches, {S} splits")
        outs.append(o.float().cpu())
    assert float((outs[0] - outs[2]).abs().max()) < 4e-3


def _word_view(exchange_buf, world, rank_rows, D):
    """Layout of the decode step's exchange: [parity][source][row][slice of 8 columns][8 + l + m]."""
    return exchange_buf[: 2 * world * rank_rows * (D // 8) * 10].view(2, world, rank_rows, D // 8, 10)


def _peer_words(exchange_buf, world, rank_rows, D, epoch, src, row0, acc, l, m):
    """Writes what rank `src` would push for rows [row0, row0 + R): words {value, epoch}."""
    words = _word_view(exchange_buf, world, rank_rows, D)
    R = acc.shape[0]
    vals = torch.cat([acc.reshape(R, D // 8, 8), l[:, None, None].expand(R, D // 8, 1),
                      m[:, None, None].expand(R, D // 8, 1)], dim=2).contiguous()       # [R, D/8, 10] f32
    bits = vals.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    words[epoch & 1, src, row0:row0 + R] = (bits | (int(epoch) << 32)).to(words.device)


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 2), (8, 5)])
def test_decode_step_exchange_with_played_peers(cuda, world, rank):
    """One sequence split over `world` ranks; this GPU is `rank` and holds its share of the
    pages, the other ranks' merged partials (computed by the oracle) are already in its exchange
    buffer.  Two steps in a row: the launch count and the buffer parity advance."""
    H, G, D, S = 8, 2, 256, 6
    L = 16 * 40 * world
    gen = torch.Generator().manual_seed(900 + world + rank)
    k, v = randn(gen, G, L, D, dtype=torch.bfloat16), randn(gen, G, L, D, dtype=torch.bfloat16)
    share = L // world
    lo = rank * share
    n_pages = share // 16
    perm = torch.randperm(n_pages, generator=gen)
    kp = torch.empty(n_pages, G, 16, D, dtype=torch.bfloat16)
    vp = torch.empty_like(kp)
    kp[perm] = k[:, lo:lo + share].reshape(G, n_pages, 16, D).permute(1, 0, 2, 3)
    vp[perm] = v[:, lo:lo + share].reshape(G, n_pages, 16, D).permute(1, 0, 2, 3)
    bt = perm.to(torch.int32)[None].to(cuda)
    time = torch.tensor([share], dtype=torch.int32, device=cuda)
    bufs = [torch.zeros(_cabi.load().g4b_exchange_buffer_bytes(world, H, D) // 8, dtype=torch.int64, device=cuda)
            for _ in range(world)]
    ex = PartialExchange(H, D, peers=bufs, rank=rank)
    po, pl, pm = _workspace(S, 1, H, D, cuda)
    for step in range(2):
        q = randn(gen, 1, H, 1, D, dtype=torch.bfloat16)
        want = orc.attention_core(q[0], k, v, scale=1 / 16)[None]
        for r in range(world):
            if r == rank:
                continue
            acc, l, m = orc.split_partials(q[0], k[:, r * share:(r + 1) * share], v[:, r * share:(r + 1) * share],
                                           scale=1 / 16, num_splits=1)
            _peer_words(bufs[rank], world, H, D, step + 1, r, 0, acc[0, :, 0], l[0, :, 0], m[0, :, 0])
        o = torch.zeros(1, H, 1, D, dtype=torch.bfloat16, device=cuda)
        fa2.decode_step(q.to(cuda), kp.to(cuda), vp.to(cuda), o, time, None, share, fa2.PHASE_DECODE, po, pl, pm,
                        exchange=ex, num_kv_splits=S, scale=1 / 16, block_tables=bt, page_size=16)
        assert_close(o, want, f"world {world} rank {rank} step {step}")
        assert ex.state.tolist()[0] == step + 1
        # what this rank pushed to a peer is its own merged partial
        acc, l, m = orc.split_partials(q[0], k[:, lo:lo + share], v[:, lo:lo + share], scale=1 / 16, num_splits=1)
        peer = (rank + 1) % world
        words = _word_view(bufs[peer], world, H, D)[(step + 1) & 1, rank].cpu()                 # [H, D/8, 10]
        assert bool(((words >> 32) == step + 1).all()), "a pushed word does not carry the launch count"
        got = (words & 0xFFFFFFFF).to(torch.int32).view(torch.float32)
        m_got, m_want = got[:, 0, 9], m[0, :, 0]
        scale_to = torch.exp2(m_got - m_want)[:, None]                  # same partial up to the choice of maximum
        assert torch.allclose(got[:, :, :8].reshape(H, D) * scale_to, acc[0, :, 0], atol=2e-2, rtol=2e-2)
    assert _cabi.device_status() == 0


def test_decode_step_absent_peer_times_out(cuda):
    """Nobody writes the peer's words: the merging CTAs give up after their bounded wait, record
    0x401, leave o alone, and the context stays usable."""
    H, G, D, S = 8, 2, 256, 2
    case = make_paged_case(950, lens=[64], H=H, G=G, dtype=torch.float16)
    bufs = [torch.zeros(_cabi.load().g4b_exchange_buffer_bytes(2, H, D) // 8, dtype=torch.int64, device=cuda)
            for _ in range(2)]
    ex = PartialExchange(H, D, peers=bufs, rank=0)
    po, pl, pm = _workspace(S, 1, H, D, cuda)
    o = torch.full((1, H, 1, D), 5.0, dtype=torch.float16, device=cuda)
    fa2.decode_step(case["q"].to(cuda), case["k_pool"].to(cuda), case["v_pool"].to(cuda), o, case["time"].to(cuda), None,
                    case["max_len"], fa2.PHASE_DECODE, po, pl, pm, exchange=ex, num_kv_splits=S, scale=1 / 16,
                    block_tables=case["block_tables"].to(cuda), page_size=16)
    assert _cabi.device_status() == 0x401
    assert bool((o == 5.0).all())
    # an ordinary call afterwards works
    o2 = torch.zeros_like(o)
    fa2.flash_attention(case["q"].to(cuda), case["k_pool"].to(cuda), case["v_pool"].to(cuda), o2, case["time"].to(cuda),
                        None, case["max_len"], fa2.PHASE_DECODE, scale=1 / 16,
                        block_tables=case["block_tables"].to(cuda), page_size=16)
    want = orc.flash_attention(case["q"], case["k_pool"], case["v_pool"], torch.zeros(1, H, 1, D), case["time"], None,
                               case["max_len"], 2, scale=1 / 16, block_tables=case["block_tables"], page_size=16)
    assert_close(o2, want, "after a timed-out exchange")
