"""Norm + rotary embedding + KV append in one launch, on the GPU through the C ABI, against
the reference's own outputs (golden vectors) and the oracle.

Tolerances: the arithmetic is fp32 on both sides, so fp32 outputs agree to a few ulp
(2e-5 abs+rel: the multiplications are grouped differently and rsqrt / sincos are different
implementations); 16-bit outputs to one ulp of that type.  Where the row is only moved
(block-table and ring indexing) the comparison is on which rows changed, bit for bit."""
from pathlib import Path

import numpy as np
import pytest
import torch

from g4b_b200.kernels.fa2 import flash_attention
from g4b_b200.kernels.rope import apply_rope, rope_norm_append
from helpers import assert_close, orc, randn

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


def load(name):
    z = np.load(GOLD / f"{name}.npz")
    return {k: (torch.from_numpy(z[k].astype(np.float32)) if z[k].ndim else z[k].item()) for k in z.files}


def ulp_tol(dtype):
    return {torch.float32: 2e-5, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dtype]


@pytest.mark.parametrize("name", ["rope_swa", "rope_global_far", "rope_d128"])
def test_apply_rope_matches_reference_golden(cuda, name):
    """The reference's signature, in place on fp32 q and k, sums of squares passed in."""
    g = load(name)
    q, k = g["q"][None].to(cuda), g["k"][None].to(cuda)
    off = torch.tensor([int(g["base_time_offset"])], dtype=torch.int32, device=cuda)
    apply_rope(q, k, g["freqs"].to(cuda), off, (q * q).sum(-1), (k * k).sum(-1), g["q_w"].to(cuda),
               g["k_w"].to(cuda), float(g["eps"]))
    assert torch.allclose(q[0].cpu(), g["q_out"], atol=2e-5, rtol=2e-5), (q[0].cpu() - g["q_out"]).abs().max()
    assert torch.allclose(k[0].cpu(), g["k_out"], atol=2e-5, rtol=2e-5), (k[0].cpu() - g["k_out"]).abs().max()


@pytest.mark.parametrize("name", ["rope_swa", "rope_global_far"])
@pytest.mark.parametrize("cache_dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_fused_matches_reference_golden(cuda, name, cache_dtype):
    """Fused form on the golden inputs: q to a separate 16-bit tensor, k and the normalised v
    into a ring cache that wraps, sums of squares computed by the kernel."""
    g = load(name)
    H, n, D = g["q"].shape
    G = g["k"].shape[0]
    T = n + 2
    base = int(g["base_time_offset"])
    q, k, v = (g[x][None].to(cuda) for x in ("q", "k", "v"))
    q_keep = q.clone()
    q_out = torch.zeros(1, H, n, D, dtype=cache_dtype, device=cuda)
    kc = torch.zeros(1, G, T, D, dtype=cache_dtype, device=cuda)
    vc = torch.zeros(1, G, T, D, dtype=cache_dtype, device=cuda)
    off = torch.tensor([base], dtype=torch.int64, device=cuda)
    rope_norm_append(q, k, v, g["freqs"].to(cuda), off, kc, vc, float(g["eps"]), q_out=q_out,
                     q_rmsnorm_w=g["q_w"].to(cuda), k_rmsnorm_w=g["k_w"].to(cuda))
    tol = ulp_tol(cache_dtype)
    assert torch.equal(q, q_keep), "q must stay untouched when q_out is given"
    assert torch.allclose(q_out[0].float().cpu(), g["q_out"], atol=tol, rtol=tol)
    rows = [(base + t) % T for t in range(n)]
    assert torch.allclose(kc[0][:, rows].float().cpu(), g["k_out"], atol=tol, rtol=tol)
    assert torch.allclose(vc[0][:, rows].float().cpu(), g["v_out"], atol=tol, rtol=tol)
    untouched = [r for r in range(T) if r not in rows]
    assert (kc[0][:, untouched] == 0).all() and (vc[0][:, untouched] == 0).all()


@pytest.mark.parametrize("in_dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,Tq", [(3, 1), (2, 19), (4, 512)])
def test_fused_ring_against_oracle(cuda, in_dtype, B, Tq):
    """Engine layout (physical [B,t,heads,D] viewed as [B,heads,t,D]), rsos passed as strided
    views, phase gate on the append but not on the rotation."""
    gen = torch.Generator().manual_seed(100 + B + Tq)
    H, G, D, T = 8, 2, 256, Tq + 40
    q_phys = randn(gen, B, Tq, H, D, dtype=in_dtype)
    k_phys = randn(gen, B, Tq, G, D, dtype=in_dtype)
    v_phys = randn(gen, B, Tq, G, D, dtype=in_dtype)
    q, k, v = (x.permute(0, 2, 1, 3) for x in (q_phys, k_phys, v_phys))
    rs = [(x.float() ** 2).sum(-1).contiguous() for x in (q_phys, k_phys, v_phys)]      # [B,t,heads]
    q_w, k_w = 1 + 0.1 * randn(gen, D), 1 + 0.1 * randn(gen, D)
    freqs = 1.0 / (10000.0 ** (torch.arange(0, D, 2) / D))
    off = torch.tensor([5, T - 3, 1000, 77][:B], dtype=torch.int32)
    phase = torch.tensor([1, 1, 2, 1][:B], dtype=torch.uint8)
    kc0, vc0 = randn(gen, B, G, T, D, dtype=torch.float16), randn(gen, B, G, T, D, dtype=torch.float16)
    want_q, want_k, want_kc, want_vc = orc.rope_norm_append(
        q, k, v, freqs, off, kc0, vc0, 1e-6, q_rsos=rs[0].permute(0, 2, 1), k_rsos=rs[1].permute(0, 2, 1),
        v_rsos=rs[2].permute(0, 2, 1), q_rmsnorm_w=q_w, k_rmsnorm_w=k_w, user_phase=phase, phase=1)

    qd, kd, vd = (x.to(cuda).permute(0, 2, 1, 3) for x in (q_phys, k_phys, v_phys))
    rsd = [x.to(cuda).permute(0, 2, 1) for x in rs]
    kc, vc = kc0.to(cuda), vc0.to(cuda)
    k_out = torch.zeros(B, G, Tq, D, dtype=torch.float32, device=cuda)
    rope_norm_append(qd, kd, vd, freqs.to(cuda), off.to(cuda), kc, vc, 1e-6, k_out=k_out, q_rsos=rsd[0],
                     k_rsos=rsd[1], v_rsos=rsd[2], q_rmsnorm_w=q_w.to(cuda), k_rmsnorm_w=k_w.to(cuda),
                     user_phase=phase.to(cuda), phase=1)
    tol = ulp_tol(in_dtype)
    assert torch.allclose(qd.float().cpu(), want_q, atol=tol, rtol=tol)        # in place, all slots
    assert torch.allclose(k_out.cpu(), want_k, atol=2e-5, rtol=2e-5)
    assert torch.allclose(kc.float().cpu(), want_kc.float(), atol=1e-3, rtol=1e-3)
    assert torch.allclose(vc.float().cpu(), want_vc.float(), atol=1e-3, rtol=1e-3)
    # rows of slots off phase, and rows that received no token, keep their bits
    same = (want_kc == kc0).all(-1)
    assert torch.equal(kc.cpu()[same], kc0[same]) and torch.equal(vc.cpu()[same], vc0[same])


@pytest.mark.parametrize("page_size", [16, 32])
def test_fused_paged_then_attention(cuda, page_size):
    """Paged caches: append a chunk through the fused kernel, then run attention on what it
    wrote and compare with the oracle end to end (bf16, the prefill kernel's input type)."""
    gen = torch.Generator().manual_seed(9)
    B, H, G, D, Tq = 2, 4, 2, 256, 150
    before = [0, 45]
    pages_per = [(b + Tq + page_size - 1) // page_size for b in before]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=gen).to(torch.int32)
    bt = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages_per):
        bt[b, :n] = perm[at:at + n]
        at += n
    q, k, v = randn(gen, B, H, Tq, D), randn(gen, B, G, Tq, D), randn(gen, B, G, Tq, D)
    k_pool0 = randn(gen, num_pages, G, page_size, D, dtype=torch.bfloat16)
    v_pool0 = randn(gen, num_pages, G, page_size, D, dtype=torch.bfloat16)
    freqs = 1.0 / (10000.0 ** (torch.arange(0, D, 2) / D))
    off = torch.tensor(before, dtype=torch.int32)
    time = off + Tq
    cw = bt.shape[1] * page_size
    want_q, _, want_kp, want_vp = orc.rope_norm_append(q, k, v, freqs, off, k_pool0, v_pool0, 1e-6,
                                                       block_tables=bt, page_size=page_size)
    o = torch.zeros(B, H, Tq, D)
    want_o = orc.flash_attention(want_q.to(torch.bfloat16), want_kp, want_vp, o, time, None, cw, 1, scale=1 / 16,
                                 block_tables=bt, page_size=page_size)

    kp, vp = k_pool0.to(cuda), v_pool0.to(cuda)
    q16 = torch.zeros(B, H, Tq, D, dtype=torch.bfloat16, device=cuda)
    rope_norm_append(q.to(cuda), k.to(cuda), v.to(cuda), freqs.to(cuda), off.to(cuda), kp, vp, 1e-6, q_out=q16,
                     block_tables=bt.to(cuda), page_size=page_size)
    assert torch.allclose(kp.float().cpu(), want_kp.float(), atol=8e-3, rtol=8e-3)
    assert torch.allclose(vp.float().cpu(), want_vp.float(), atol=8e-3, rtol=8e-3)
    same = (want_kp == k_pool0).all(-1)
    assert torch.equal(kp.cpu()[same], k_pool0[same]), "pages outside the block tables were written"
    od = torch.zeros(B, H, Tq, D, dtype=torch.bfloat16, device=cuda)
    flash_attention(q16, kp, vp, od, time.to(cuda), None, cw, 1, scale=1 / 16, block_tables=bt.to(cuda),
                    page_size=page_size)
    # K, V and q each carry one bf16 rounding that may fall differently on the two sides (checked
    # row by row above), so the attention is compared with the oracle's over the rows the GPU
    # holds, at the tolerance of every other parity test
    want_gpu_rows = orc.flash_attention(q16.cpu(), kp.cpu(), vp.cpu(), o, time, None, cw, 1, scale=1 / 16,
                                        block_tables=bt, page_size=page_size)
    assert_close(od, want_gpu_rows, "attention over the fused append")
    # and stays near the oracle's end-to-end answer (three independent bf16 roundings apart)
    assert_close(od, want_o, "attention over the fused append, oracle rows", abs_tol=8e-3, rel_tol=2e-2)


def test_no_rotation_and_no_norm_moves_bits(cuda):
    """rope_freqs absent and norms off: the call degenerates to a cast-and-append, bit-exact."""
    gen = torch.Generator().manual_seed(5)
    B, H, G, D, Tq, T = 2, 2, 2, 128, 5, 9
    q, k, v = (randn(gen, B, h, Tq, D, dtype=torch.float16) for h in (H, G, G))
    kc0, vc0 = randn(gen, B, G, T, D, dtype=torch.float16), randn(gen, B, G, T, D, dtype=torch.float16)
    off = torch.tensor([7, 2], dtype=torch.int32)
    want_k = orc.add_kv_to_cache(k, kc0, off, 0.0)
    want_v = orc.add_kv_to_cache(v, vc0, off, 0.0)
    qd, kc, vc = q.to(cuda), kc0.to(cuda), vc0.to(cuda)
    rope_norm_append(qd, k.to(cuda), v.to(cuda), None, off.to(cuda), kc, vc, 0.0, norm_qk=False, norm_v=False)
    assert torch.equal(kc.cpu(), want_k) and torch.equal(vc.cpu(), want_v) and torch.equal(qd.cpu(), q)


def test_bad_arguments_raise(cuda):
    D = 256
    q = torch.zeros(1, 4, 2, D, device=cuda)
    k = torch.zeros(1, 2, 2, D, device=cuda)
    off = torch.zeros(1, dtype=torch.int32, device=cuda)
    freqs = torch.zeros(D // 2, device=cuda)
    with pytest.raises(ValueError):       # frequencies must cover D/2 pairs (rope.py:147)
        apply_rope(q, k, freqs[:64], off, None, None, None, None, 1e-6)
    with pytest.raises(ValueError):       # k must share batch, tokens and head dim with q
        apply_rope(q, k[:, :, :1], freqs, off, None, None, None, None, 1e-6)
    with pytest.raises(ValueError):       # v without a cache to put it in
        rope_norm_append(q, k, k.clone(), freqs, off, None, None, 1e-6)
    with pytest.raises(ValueError):
        apply_rope(q.half(), k, freqs, off, None, None, None, None, 1e-6)


@pytest.mark.parametrize("D,H,G,B,Tq", [(512, 2, 1, 2, 7), (64, 4, 4, 1, 33), (128, 5, 1, 1, 2400), (512, 3, 1, 1, 3300)])
def test_other_head_dims_and_head_counts(cuda, D, H, G, B, Tq):
    """Head dims 64 / 128 / 512 (the two-pass form of the kernel), head counts that do not fill
    the four-row batches, and both work splits (one head per warp; all heads of a token per
    warp above 16384 rows)."""
    gen = torch.Generator().manual_seed(D + H + Tq)
    T = Tq + 5
    q, k, v = randn(gen, B, H, Tq, D), randn(gen, B, G, Tq, D), randn(gen, B, G, Tq, D)
    q_w, k_w = 1 + 0.1 * randn(gen, D), 1 + 0.1 * randn(gen, D)
    freqs = 1.0 / (10000.0 ** (torch.arange(0, D, 2) / D))
    off = torch.tensor([3, T - 2][:B], dtype=torch.int32)
    kc0, vc0 = randn(gen, B, G, T, D, dtype=torch.bfloat16), randn(gen, B, G, T, D, dtype=torch.bfloat16)
    want_q, want_k, want_kc, want_vc = orc.rope_norm_append(q, k, v, freqs, off, kc0, vc0, 1e-6, q_rmsnorm_w=q_w,
                                                            k_rmsnorm_w=k_w)
    qd, kd = q.to(cuda), k.to(cuda)
    kc, vc = kc0.to(cuda), vc0.to(cuda)
    k_out = torch.zeros(B, G, Tq, D, device=cuda)
    rope_norm_append(qd, kd, v.to(cuda), freqs.to(cuda), off.to(cuda), kc, vc, 1e-6, k_out=k_out,
                     q_rmsnorm_w=q_w.to(cuda), k_rmsnorm_w=k_w.to(cuda))
    assert torch.allclose(qd.cpu(), want_q, atol=2e-5, rtol=2e-5)             # in place, fp32
    assert torch.allclose(k_out.cpu(), want_k, atol=2e-5, rtol=2e-5)
    assert torch.equal(kd.cpu(), k)                                           # k itself is left alone when it has a destination
    assert torch.allclose(kc.float().cpu(), want_kc.float(), atol=8e-3, rtol=8e-3)
    assert torch.allclose(vc.float().cpu(), want_vc.float(), atol=8e-3, rtol=8e-3)


def test_reference_rope_script_case(cuda):
    """The case of the reference's rope comparison script (tests/compare_scripts/test_rope.py:
    B, h, T, k = 1, 48, 1, 512; q and k of the same shape; position 1000; frequency base 1e5;
    frequency scales of 1 for the first half of the pairs and -inf for the rest, i.e. those
    pairs are not rotated), through apply_rope and against the oracle."""
    gen = torch.Generator().manual_seed(48)
    B, h, T, k = 1, 48, 1, 512
    q, kk = randn(gen, B, h, T, k), randn(gen, B, h, T, k)
    q_w, k_w = randn(gen, k), randn(gen, k)
    scales = torch.cat([torch.ones(k // 4), torch.full((k // 4,), float("-inf"))])
    freqs = 1.0 / (100000.0 ** (torch.arange(0, k, 2) / k)) / scales
    off = torch.tensor([1000], dtype=torch.int64)
    pos = off[:, None] + torch.arange(T)[None]
    want_q = orc.rope_norm(q, pos, freqs, rsos=(q * q).sum(-1), weight=q_w, eps=1e-6)
    want_k = orc.rope_norm(kk, pos, freqs, rsos=(kk * kk).sum(-1), weight=k_w, eps=1e-6)
    qd, kd = q.to(cuda), kk.to(cuda)
    apply_rope(qd, kd, freqs.to(cuda), off.to(cuda), (qd * qd).sum(-1), (kd * kd).sum(-1), q_w.to(cuda), k_w.to(cuda), 1e-6)
    assert torch.allclose(qd.cpu(), want_q, atol=5e-5, rtol=5e-5), (qd.cpu() - want_q).abs().max()
    assert torch.allclose(kd.cpu(), want_k, atol=5e-5, rtol=5e-5), (kd.cpu() - want_k).abs().max()
    # the unrotated pairs are exactly the normalised inputs
    inv = torch.rsqrt((q * q).sum(-1) / k + 1e-6)[..., None]
    assert torch.allclose(qd.cpu()[..., k // 4: k // 2], (q * (inv * q_w))[..., k // 4: k // 2], atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("D", [64, 200, 256, 512])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,Tq,paged", [(5, 1, True), (3, 6, False), (2, 2100, True), (1, 1500, False)])
def test_engine_configuration_variants(cuda, D, dtype, B, Tq, paged):
    """The configuration the engine runs (gemma4e.py:564-592): f32 q/k/v, q and k normed with
    weights and rotated, v normed, q into a 16-bit q_out, k and v into 16-bit caches only.  The
    kernel has compile-time variants for exactly this; here they run at head dims on and off
    their full-width case, one row per warp (few rows) and a token per warp (many), ring and
    pages, with and without V norm, far positions, and a slot off phase."""
    gen = torch.Generator().manual_seed(D + Tq)
    H, G = 8, 2
    q, k, v = (randn(gen, B, Tq, h, D).permute(0, 2, 1, 3) for h in (H, G, G))
    q_w, k_w = 1 + 0.1 * randn(gen, D), 1 + 0.1 * randn(gen, D)
    freqs = 1.0 / (10000.0 ** (torch.arange(0, D, 2) / D))
    before = [0, 100000, 17, 3, 50000][:B]
    off = torch.tensor(before, dtype=torch.int32)
    phase = torch.tensor([1, 1, 2, 1, 1][:B], dtype=torch.uint8)
    norm_v = Tq != 6
    if paged:
        page = 16
        pages_per = [(b + Tq + page - 1) // page for b in before]
        n_pages = sum(p - b // page for p, b in zip(pages_per, before)) + 2      # only the pages the new rows touch
        perm = torch.randperm(n_pages, generator=gen).to(torch.int32)
        bt = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
        at = 0
        for b, (n, first) in enumerate(zip(pages_per, before)):
            lo = first // page
            bt[b, lo:n] = perm[at:at + n - lo]
            at += n - lo
        kc0, vc0 = randn(gen, n_pages, G, page, D, dtype=dtype), randn(gen, n_pages, G, page, D, dtype=dtype)
        extra = dict(block_tables=bt, page_size=page)
    else:
        T = Tq + 9
        kc0, vc0 = randn(gen, B, G, T, D, dtype=dtype), randn(gen, B, G, T, D, dtype=dtype)
        extra = {}
    want_q, _, want_kc, want_vc = orc.rope_norm_append(q, k, v, freqs, off, kc0, vc0, 1e-6, q_rmsnorm_w=q_w,
                                                       k_rmsnorm_w=k_w, norm_v=norm_v, user_phase=phase, phase=1, **extra)
    kc, vc = kc0.to(cuda), vc0.to(cuda)
    q_out = torch.zeros(B, H, Tq, D, dtype=dtype, device=cuda)
    qd = q.to(cuda)
    dev_extra = {key: (val.to(cuda) if torch.is_tensor(val) else val) for key, val in extra.items()}
    rope_norm_append(qd, k.to(cuda), v.to(cuda), freqs.to(cuda), off.to(cuda), kc, vc, 1e-6, q_out=q_out,
                     q_rmsnorm_w=q_w.to(cuda), k_rmsnorm_w=k_w.to(cuda), norm_v=norm_v, user_phase=phase.to(cuda),
                     phase=1, **dev_extra)
    tol = ulp_tol(dtype)
    assert torch.equal(qd.cpu(), q), "q must stay untouched when q_out is given"
    assert torch.allclose(q_out.float().cpu(), want_q, atol=tol, rtol=tol)
    assert torch.allclose(kc.float().cpu(), want_kc.float(), atol=tol, rtol=tol)
    assert torch.allclose(vc.float().cpu(), want_vc.float(), atol=tol, rtol=tol)
    same = (want_kc == kc0).all(-1)
    assert torch.equal(kc.cpu()[same], kc0[same]) and torch.equal(vc.cpu()[same], vc0[same])
