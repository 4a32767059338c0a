"""Pins the CPU oracle to the reference: committed golden vectors produced by the
reference's own LayerKVCache (tests/golden/make_golden.py) and, where the reference checkout
is mounted, live comparisons on fresh seeded inputs."""
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import orc
from oracle import ref_loader

GOLD = Path(__file__).resolve().parent / "golden"
CASES = ["prefill_causal", "prefill_causal_unscaled", "prefill_swa", "prefill_chunked",
         "decode_global", "decode_swa"]


def load(name):
    z = np.load(GOLD / f"{name}.npz")
    return {k: (torch.from_numpy(z[k].astype(np.float32)) if z[k].ndim else z[k].item()) for k in z.files}


def oracle_through_ring(g, T):
    """Feeds the golden K/V through the oracle's ring append, then attends like the engine:
    one slot, cache_offsets = tokens before the chunk, time = tokens after it
    (g4b/scheduler.py:158-172,199-203)."""
    G, n_all, D = g["k_all"].shape
    Tq = int(g["last_chunk"])
    k_cache = torch.zeros(1, G, T, D)
    v_cache = torch.zeros(1, G, T, D)
    off = torch.tensor([0])
    k_cache = orc.add_kv_to_cache(g["k_all"][None], k_cache, off, 1e-6)
    v_cache = orc.add_kv_to_cache(g["v_all"][None], v_cache, off, 1e-6)
    time = torch.tensor([n_all], dtype=torch.int32)
    is_swa = bool(g["is_swa"])
    window = int(g["window"])
    # a sliding-window layer's cache exposes window + Tq - 1 keys (g4b/models/gemma4e.py:704-705)
    ctx_window = min(T, window + Tq - 1) if is_swa else T
    o = torch.zeros(1, g["q"].shape[0], Tq, D)
    return orc.flash_attention(g["q"][None], k_cache, v_cache, o, time, None, ctx_window, 1,
                               scale=float(g["scale"]), sliding_window=window if is_swa else None)[0]


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference_golden(name):
    g = load(name)
    got = oracle_through_ring(g, T=64)
    assert torch.allclose(got, g["out"], atol=2e-6, rtol=1e-5), (got - g["out"]).abs().max()


@pytest.mark.parametrize("name", CASES)
def test_oracle_golden_ring_wrapped(name):
    """Same golden, but the ring buffer is barely long enough, so the stored rows wrap."""
    g = load(name)
    n_all = g["k_all"].shape[1]
    Tq = int(g["last_chunk"])
    if not bool(g["is_swa"]):
        pytest.skip("a global layer's ring never wraps while the context fits")
    T = int(g["window"]) + Tq - 1
    if T >= n_all:
        pytest.skip("the chunk is as long as the context: nothing wraps")
    got = oracle_through_ring(g, T=T)
    assert torch.allclose(got, g["out"], atol=2e-6, rtol=1e-5), (got - g["out"]).abs().max()


def test_oracle_config1_rows():
    """Rows of the benchmark's CPU configuration (B1 S512 H8 G2 D256 fp32, scale 1/16)."""
    z = np.load(GOLD / "config1_rows.npz")
    gen = torch.Generator().manual_seed(int(z["seed"]))
    rnd = lambda *s: torch.randn(*s, generator=gen).to(torch.float16).to(torch.float32)
    q, k, v = rnd(1, 8, 512, 256), rnd(1, 2, 512, 256), rnd(1, 2, 512, 256)
    checksum = float(q.double().sum() + k.double().sum() + v.double().sum())
    if abs(checksum - float(z["in_checksum"])) > 1e-6:
        pytest.skip("this torch build draws different random numbers than the one that made the fixture")
    out = orc.attention_core(q[0], k[0], v[0], scale=1 / 16)
    rows = z["rows"]
    assert torch.allclose(out[:, rows], torch.from_numpy(z["out_rows"]), atol=2e-6, rtol=1e-5)


@pytest.mark.skipif(not ref_loader.available(), reason="reference checkout not mounted")
@pytest.mark.parametrize("is_swa,n_prefill,n_decode", [(False, 33, 3), (True, 50, 2), (True, 9, 0)])
def test_oracle_matches_live_reference(is_swa, n_prefill, n_decode):
    """Drives the reference's LayerKVCache and the oracle side by side through a prefill and
    some decode steps."""
    H, G, D, W, ctx = 4, 2, 64, 16, 128
    gen = torch.Generator().manual_seed(7)
    cache = ref_loader.make_layer_cache(heads=H, kv_heads=G, head_dim=D, context_length=ctx,
                                        sliding_window=W, is_swa=is_swa)
    T = 96
    k_cache = torch.zeros(1, G, T, D)
    v_cache = torch.zeros(1, G, T, D)
    total = 0
    steps = [("prefill", n_prefill)] + [("decode", 1)] * n_decode
    for phase, n in steps:
        (cache.set_prefill if phase == "prefill" else cache.set_decode)()
        k, v, q = (torch.randn(1, G, n, D, generator=gen), torch.randn(1, G, n, D, generator=gen),
                   torch.randn(1, H, n, D, generator=gen))
        cache.add(k, v)
        want = cache.retrieve(q * 0.125)
        off = torch.tensor([total])
        k_cache = orc.add_kv_to_cache(k, k_cache, off, 1e-6)
        v_cache = orc.add_kv_to_cache(v, v_cache, off, 1e-6)
        total += n
        ctx_window = min(T, W + n - 1) if is_swa else T
        got = orc.flash_attention(q, k_cache, v_cache, torch.zeros(1, H, n, D), torch.tensor([total]), None,
                                  ctx_window, 1, scale=0.125, sliding_window=W if is_swa else None)
        assert torch.allclose(got, want, atol=2e-6, rtol=1e-5), (phase, n, (got - want).abs().max())


def test_oracle_combine_equals_unsplit():
    """Splitting the key range and merging (fa2.py:438-472, 618-626) is the identity."""
    gen = torch.Generator().manual_seed(3)
    H, G, D, Tk = 8, 2, 256, 333
    q = torch.randn(H, 1, D, generator=gen)
    k = torch.randn(G, Tk, D, generator=gen)
    v = torch.randn(G, Tk, D, generator=gen)
    full = orc.attention_core(q, k, v, scale=1 / 16)
    for S in (1, 2, 7, 16, 40):   # 40 > number of 16-key blocks: trailing splits are empty
        acc, l, m = orc.split_partials(q, k, v, scale=1 / 16, num_splits=S)
        got = orc.combine_partials(acc[:, None], l[:, None], m[:, None], S)[0]
        assert torch.allclose(got, full, atol=1e-5, rtol=1e-4)


def test_oracle_paged_equals_ring():
    gen = torch.Generator().manual_seed(5)
    H, G, D, ps = 4, 2, 64, 16
    lens = [37, 16, 1]
    pages = [3, 1, 1]
    perm = torch.randperm(8, generator=gen)
    bt = torch.zeros(3, 3, dtype=torch.int32)
    bt[0] = perm[:3]; bt[1, 0] = perm[3]; bt[2, 0] = perm[4]
    pool_k = torch.randn(8, G, ps, D, generator=gen)
    pool_v = torch.randn(8, G, ps, D, generator=gen)
    q = torch.randn(3, H, 1, D, generator=gen)
    got = orc.flash_attention(q, pool_k, pool_v, torch.zeros(3, H, 1, D), torch.tensor(lens), None, 48, 2,
                              block_tables=bt, page_size=ps, scale=0.125)
    for b, n in enumerate(lens):
        k = orc.gather_pages(pool_k, bt[b], n, ps)
        v = orc.gather_pages(pool_v, bt[b], n, ps)
        assert torch.allclose(got[b], orc.attention_core(q[b], k, v, scale=0.125), atol=1e-6)
    assert pages == [(n + ps - 1) // ps for n in lens]


def test_oracle_add_kv_ring_and_paged_bit_exact():
    """The append moves bits: wrap-around ring (the reference's own case B,G,t,T,D = 2,4,7,17,256
    with offsets [15, 3], tests/compare_scripts/test_add_kv.py:19,29) and paged destinations."""
    gen = torch.Generator().manual_seed(9)
    B, G, t, T, D = 2, 4, 7, 17, 256
    x = torch.randn(B, G, t, D, generator=gen)
    cache = torch.randn(B, G, T, D, generator=gen)
    off = torch.tensor([15, 3])
    out = orc.add_kv_to_cache(x, cache, off, 1e-6)
    for b in range(B):
        for tt in range(t):
            assert torch.equal(out[b, :, (int(off[b]) + tt) % T], x[b, :, tt])
    untouched = torch.ones(B, T, dtype=torch.bool)
    for b in range(B):
        untouched[b, (int(off[b]) + torch.arange(t)) % T] = False
    assert torch.equal(out.permute(0, 2, 1, 3)[untouched], cache.permute(0, 2, 1, 3)[untouched])
    # rms-normalised variant against the reference test's formula (test_add_kv.py:54-59)
    rsos = (x * x).sum(-1)
    out_n = orc.add_kv_to_cache(x, cache, off, 1e-6, rsos)
    x_norm = x / (rsos.unsqueeze(-1) / D + 1e-6).sqrt()
    assert torch.allclose(out_n[0, :, 15], x_norm[0, :, 0], rtol=1e-6, atol=1e-7)


def test_oracle_advance_and_policy():
    inp = np.zeros((1, 4), np.int32)
    out_tok = np.array([[5], [6], [7], [8]], np.int32)
    off = np.array([10, 20, 30, 40], np.int32)
    tim = off + 1
    ph = np.array([2, 1, 0, 2], np.uint8)
    i2, o2, t2 = orc.advance_decode_state(inp, out_tok, off, tim, ph)
    assert i2.tolist() == [[5, 0, 0, 8]] and o2.tolist() == [11, 20, 30, 41] and t2.tolist() == [12, 21, 31, 42]
    # fa2.py:204-212
    assert [orc.select_kv_splits(w, 16, 2, 1) for w in (1024, 4096, 4097, 8192, 32767, 32768)] == [1, 1, 4, 8, 8, 16]
    assert orc.select_kv_splits(65536, 4, 2, 1) == 4
    assert orc.select_kv_splits(65536, 16, 1, 1) == 1 and orc.select_kv_splits(65536, 16, 2, 2) == 1


ROPE_CASES = ["rope_swa", "rope_global_far", "rope_d128"]


@pytest.mark.parametrize("name", ROPE_CASES)
def test_oracle_rope_norm_matches_reference_golden(name):
    """q_norm/k_norm/v_norm + RoPE of the reference (reference_impl.py:219-233) against the
    oracle's restatement of the kernel's formulation (g4b/kernels/rope.py:22-39)."""
    g = load(name)
    n = g["q"].shape[1]
    pos = (int(g["base_time_offset"]) + torch.arange(n))[None]
    eps = float(g["eps"])
    q = orc.rope_norm(g["q"][None], pos, g["freqs"], weight=g["q_w"], eps=eps)[0]
    k = orc.rope_norm(g["k"][None], pos, g["freqs"], weight=g["k_w"], eps=eps)[0]
    v = orc.rope_norm(g["v"][None], pos, None, eps=eps)[0]
    # fp32 throughout on both sides; the orders of the multiplications differ
    assert torch.allclose(q, g["q_out"], atol=2e-5, rtol=2e-5), (q - g["q_out"]).abs().max()
    assert torch.allclose(k, g["k_out"], atol=2e-5, rtol=2e-5), (k - g["k_out"]).abs().max()
    assert torch.allclose(v, g["v_out"], atol=2e-5, rtol=2e-5), (v - g["v_out"]).abs().max()


@pytest.mark.skipif(not ref_loader.available(), reason="reference checkout not mounted")
def test_oracle_rope_norm_append_live_against_reference():
    """Fresh inputs through the reference's norms, RoPE and LayerKVCache.add, against the
    oracle's fused restatement writing a ring cache."""
    gen = torch.Generator().manual_seed(77)
    G, H, D, n = 2, 4, 256, 12
    q_w = 1 + 0.1 * torch.randn(D, generator=gen)
    k_w = 1 + 0.1 * torch.randn(D, generator=gen)
    rope, q_norm, k_norm, v_norm = ref_loader.make_rope_and_norms(head_dim=D, is_swa=True, freq_base=10000.0,
                                                                  eps=1e-6, q_weight=q_w, k_weight=k_w)
    cache = ref_loader.make_layer_cache(heads=H, kv_heads=G, head_dim=D, context_length=64, sliding_window=16,
                                        is_swa=False)
    q, k, v = (torch.randn(1, h, n, D, generator=gen) for h in (H, G, G))
    cache.set_prefill()
    base = cache.base_time_offset
    (k_ref,) = rope(k_norm(k), base_time_offset=base)
    (q_ref,) = rope(q_norm(q), base_time_offset=base)
    cache.add(k_ref, v_norm(v))
    out_ref = cache.retrieve(q_ref / 16)
    kc, vc = torch.zeros(1, G, 32, D), torch.zeros(1, G, 32, D)
    q2, k2, kc, vc = orc.rope_norm_append(q, k, v, rope.freqs, torch.tensor([base]), kc, vc, 1e-6,
                                          q_rmsnorm_w=q_w, k_rmsnorm_w=k_w)
    assert torch.allclose(q2, q_ref, atol=2e-5, rtol=2e-5)
    assert torch.allclose(kc[0, :, :n], k_ref[0], atol=2e-5, rtol=2e-5)
    o = torch.zeros(1, H, n, D)
    out = orc.flash_attention(q2, kc, vc, o, torch.tensor([n], dtype=torch.int32), None, 32, 1, scale=1 / 16)
    assert torch.allclose(out, out_ref, atol=1e-5, rtol=1e-4)
