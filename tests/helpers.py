"""Seeded input builders shared by the tests (CPU tensors; GPU tests move them over)."""
from __future__ import annotations

import torch

from oracle import attention_oracle as orc

TOL_ABS, TOL_REL = 2e-3, 1e-2   # |a-b| <= TOL_ABS + TOL_REL*|b| for f16/bf16 outputs


def assert_close(got: torch.Tensor, want: torch.Tensor, what: str = "", abs_tol=TOL_ABS, rel_tol=TOL_REL):
    got = got.detach().to("cpu", torch.float32)
    want = want.detach().to("cpu", torch.float32)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite values in the result"
    err = (got - want).abs()
    bound = abs_tol + rel_tol * want.abs()
    worst = (err - bound).max().item()
    assert worst <= 0, f"{what}: max abs err {err.max().item():.3e}, exceeds tolerance by {worst:.3e}"


def randn(gen, *shape, dtype=torch.float32):
    return torch.randn(*shape, generator=gen, dtype=torch.float32).to(dtype)


def make_ring_case(seed, *, B, H, G, Tq, T, D=256, dtype=torch.bfloat16, times=None, ctx_window=None):
    """q [B,H,Tq,D] as a strided view of physical [B,Tq,H,D] (like the engine's scratchpads,
    g4b/models/gemma4e.py:1031-1033), ring caches [B,G,T,D] filled with data everywhere."""
    gen = torch.Generator().manual_seed(seed)
    q_phys = randn(gen, B, Tq, H, D, dtype=dtype)
    k = randn(gen, B, G, T, D, dtype=dtype)
    v = randn(gen, B, G, T, D, dtype=dtype)
    ctx_window = T if ctx_window is None else ctx_window
    if times is None:
        times = [ctx_window if b % 2 == 0 else ctx_window + 17 for b in range(B)]   # test_fa2.py:286-290
    return dict(q_phys=q_phys, q=q_phys.permute(0, 2, 1, 3), k=k, v=v,
                time=torch.tensor(times, dtype=torch.int32), ctx_window=ctx_window)


def make_paged_case(seed, *, lens, H, G, D=256, page_size=16, dtype=torch.float16, extra_pages=3):
    """Decode inputs over a shuffled page pool.  lens[b] = context length incl. the new token."""
    gen = torch.Generator().manual_seed(seed)
    B = len(lens)
    pages_per = [(n + page_size - 1) // page_size for n in lens]
    num_pages = sum(pages_per) + extra_pages
    perm = torch.randperm(num_pages, generator=gen)
    max_pages = max(pages_per)
    bt = torch.full((B, max_pages), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages_per):
        bt[b, :n] = perm[at:at + n].to(torch.int32)
        at += n
    k_pool = randn(gen, num_pages, G, page_size, D, dtype=dtype)
    v_pool = randn(gen, num_pages, G, page_size, D, dtype=dtype)
    q = randn(gen, B, H, 1, D, dtype=dtype)
    return dict(q=q, k_pool=k_pool, v_pool=v_pool, block_tables=bt,
                time=torch.tensor(lens, dtype=torch.int32), page_size=page_size, max_len=max_pages * page_size)


__all__ = ["orc", "assert_close", "randn", "make_ring_case", "make_paged_case", "TOL_ABS", "TOL_REL"]
