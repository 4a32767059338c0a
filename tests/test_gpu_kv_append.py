"""KV-cache append and decode-state advance on the GPU, through the C ABI, against the
oracle: bit-exact for the plain path, block tables and the int32 state."""
import pytest
import torch

from g4b_b200.kernels.add_kv_to_cache import add_kv_to_cache
from g4b_b200.kernels.advance_decode_state import advance_decode_state
from helpers import orc, randn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("x_dtype,c_dtype", [
    (torch.float32, torch.float32), (torch.float32, torch.float16), (torch.float32, torch.bfloat16),
    (torch.float16, torch.float16), (torch.bfloat16, torch.bfloat16), (torch.float16, torch.bfloat16),
])
@pytest.mark.parametrize("off_dtype", [torch.int32, torch.int64])
def test_ring_append_wraps_bit_exact(cuda, x_dtype, c_dtype, off_dtype):
    # the reference's own case: B,G,t,T,D = 2,4,7,17,256, offsets [15, 3] (test_add_kv.py:19,29)
    gen = torch.Generator().manual_seed(1)
    B, G, t, T, D = 2, 4, 7, 17, 256
    x_phys = randn(gen, B, t, G, D, dtype=x_dtype)        # engine layout [B,t,G,D] (gemma4e.py:1031-1033)
    x = x_phys.permute(0, 2, 1, 3)
    cache = randn(gen, B, G, T, D, dtype=c_dtype)
    off = torch.tensor([15, 3], dtype=off_dtype)
    want = orc.add_kv_to_cache(x, cache, off, 1e-6)
    cache_d = cache.to(cuda)
    add_kv_to_cache(x_phys.to(cuda).permute(0, 2, 1, 3), cache_d, off.to(cuda), 1e-6)
    assert torch.equal(cache_d.cpu().view(torch.uint8), want.view(torch.uint8))


@pytest.mark.parametrize("c_dtype", [torch.float32, torch.float16])
def test_ring_append_rmsnorm(cuda, c_dtype):
    # V-norm variant (add_kv_to_cache.py:148-151); rsqrt is approximate on both sides
    gen = torch.Generator().manual_seed(2)
    B, G, t, T, D = 2, 4, 7, 17, 256
    x = randn(gen, B, G, t, D)
    rsos_phys = (x * x).sum(-1).permute(0, 2, 1).contiguous()   # [B,t,G] -> strided [B,G,t] view
    cache = randn(gen, B, G, T, D, dtype=c_dtype)
    off = torch.tensor([15, 3], dtype=torch.int32)
    want = orc.add_kv_to_cache(x, cache, off, 1e-6, rsos_phys.permute(0, 2, 1))
    cache_d = cache.to(cuda)
    add_kv_to_cache(x.to(cuda), cache_d, off.to(cuda), 1e-6, rsos_phys.to(cuda).permute(0, 2, 1))
    got = cache_d.cpu().float()
    tol = 2e-6 if c_dtype == torch.float32 else 1e-3   # 1 ulp of the cache dtype
    assert torch.allclose(got, want.float(), rtol=tol, atol=tol)


def test_append_skips_slots_off_phase(cuda):
    gen = torch.Generator().manual_seed(3)
    B, G, t, T, D = 5, 2, 3, 32, 256
    x = randn(gen, B, G, t, D, dtype=torch.float16)
    cache = randn(gen, B, G, T, D, dtype=torch.float16)
    off = torch.tensor([0, 30, 5, 31, 8], dtype=torch.int32)
    phase = torch.tensor([1, 2, 0, 1, 2], dtype=torch.uint8)
    for ph in (1, 2):
        want = orc.add_kv_to_cache(x, cache, off, 1e-6, None, phase, ph)
        cache_d = cache.to(cuda)
        add_kv_to_cache(x.to(cuda), cache_d, off.to(cuda), 1e-6, None, phase.to(cuda), ph)
        assert torch.equal(cache_d.cpu(), want)


@pytest.mark.parametrize("t,page_size", [(1, 16), (7, 16), (40, 16), (33, 32)])
def test_paged_append_bit_exact(cuda, t, page_size):
    gen = torch.Generator().manual_seed(4)
    B, G, D = 3, 2, 256
    offs = [0, page_size - 1, 3 * page_size + 5]
    pages_per = [(o + t + page_size - 1) // page_size for o in offs]
    num_pages = sum(pages_per) + 2
    perm = torch.randperm(num_pages, generator=gen).to(torch.int32)
    bt = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages_per):
        bt[b, :n] = perm[at:at + n]
        at += n
    x = randn(gen, B, G, t, D, dtype=torch.float32)
    pool = randn(gen, num_pages, G, page_size, D, dtype=torch.float16)
    off = torch.tensor(offs, dtype=torch.int32)
    want = orc.add_kv_to_cache(x, pool, off, 1e-6, block_tables=bt, page_size=page_size)
    pool_d = pool.to(cuda)
    add_kv_to_cache(x.to(cuda), pool_d, off.to(cuda), 1e-6, block_tables=bt.to(cuda), page_size=page_size)
    assert torch.equal(pool_d.cpu(), want)
    # exactly B*t rows per head changed
    changed = (pool_d.cpu() != pool).any(-1).sum().item()
    assert changed == B * G * t


def test_paged_append_refuses_bad_table_entry(cuda):
    """A table entry outside the pool is reported through the status word, never followed."""
    from g4b_b200 import _cabi
    x = torch.ones(1, 2, 1, 256, device=cuda)
    pool = torch.zeros(4, 2, 16, 256, dtype=torch.float16, device=cuda)
    bt = torch.tensor([[99]], dtype=torch.int32, device=cuda)
    add_kv_to_cache(x, pool, torch.zeros(1, dtype=torch.int32, device=cuda), 1e-6, block_tables=bt)
    assert _cabi.device_status() == 0x102
    assert pool.abs().sum().item() == 0


def test_prefill_sized_append(cuda):
    """Whole-prompt append (B4, G2, 8192 tokens): every row lands where the index formula says."""
    gen = torch.Generator().manual_seed(5)
    B, G, t, T, D = 4, 2, 8192, 8192, 256
    x = randn(gen, B, t, G, D, dtype=torch.bfloat16).to(cuda)
    cache = torch.zeros(B, G, T, D, dtype=torch.bfloat16, device=cuda)
    off = torch.tensor([0, 100, 8191, 4096], dtype=torch.int32, device=cuda)
    add_kv_to_cache(x.permute(0, 2, 1, 3), cache, off, 1e-6)
    for b in range(B):
        rolled = torch.roll(x[b].permute(1, 0, 2), shifts=int(off[b]), dims=1)
        assert torch.equal(cache[b], rolled)


def test_advance_decode_state_bit_exact(cuda):
    gen = torch.Generator().manual_seed(6)
    B = 300
    inp = torch.randint(0, 1000, (2, B), generator=gen, dtype=torch.int32)
    out_tok = torch.randint(0, 1000, (B, 3), generator=gen, dtype=torch.int32)
    off = torch.randint(0, 1 << 20, (B,), generator=gen, dtype=torch.int32)
    tim = off + 1
    ph = torch.randint(0, 3, (B,), generator=gen).to(torch.uint8)
    want = orc.advance_decode_state(inp.numpy(), out_tok.numpy(), off.numpy(), tim.numpy(), ph.numpy())
    d = [t.to(cuda) for t in (inp, out_tok, off, tim, ph)]
    advance_decode_state(*d)
    assert d[0].cpu().numpy().tolist() == want[0].tolist()
    assert d[2].cpu().numpy().tolist() == want[1].tolist()
    assert d[3].cpu().numpy().tolist() == want[2].tolist()
    assert torch.equal(d[1].cpu(), out_tok)
