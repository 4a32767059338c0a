"""Cross-GPU split-KV merge kernel on ONE GPU: the other ranks' part is played by the test,
which writes their merged partials (8-byte words: value, launch count) into this rank's
exchange buffer BEFORE the launch (so the kernel never waits for another kernel), gives the
kernel local tensors in place of the peers' memory, and checks both what the kernel merged
and what it pushed."""
import pytest
import torch

from g4b_b200.dist import PartialExchange
from helpers import orc, randn

pytestmark = pytest.mark.gpu
COLS = 32


def merged_partial(po, pl, pm):
    """The oracle's merge (fa2.py:618-626) stopped before the division: (acc, l, m) of all splits."""
    m = pm.max(0).values
    w = torch.where(torch.isinf(pm), torch.zeros_like(pm), torch.exp2(pm - m))
    return (po * w[..., None]).sum(0), (pl * w).sum(0), m


def new_buffers(cuda, world, rows, slices):
    """One zeroed exchange buffer per rank, of the size the library asks for; the merge kernel
    uses its head as [parity, source rank, row, slice, 34 words] of int64."""
    from g4b_b200 import _cabi

    n = _cabi.load().g4b_exchange_buffer_bytes(world, rows, slices * COLS) // 8
    assert n >= 2 * world * rows * slices * (COLS + 2)
    return [torch.zeros(n, dtype=torch.int64, device=cuda) for _ in range(world)]


def words(buf, world, rows, slices):
    """The buffer as int32 [2, world, rows, slices, 34, 2]: [..., 0] the value's bits, [..., 1] the count."""
    return buf[: 2 * world * rows * slices * (COLS + 2)].view(torch.int32).view(2, world, rows, slices, COLS + 2, 2)


def deliver(buf, world, rows, slices, par, r, merged, epoch, cuda):
    """Writes rank r's merged partial into a buffer the way rank r's kernel would."""
    acc, l, m = merged
    w = words(buf, world, rows, slices)
    piece = torch.cat([acc.reshape(rows, slices, COLS), l.reshape(rows, 1, 1).expand(rows, slices, 1),
                       m.reshape(rows, 1, 1).expand(rows, slices, 1)], -1).contiguous()
    w[par, r, :, :, :, 0] = piece.view(torch.int32).to(cuda)
    w[par, r, :, :, :, 1] = epoch


def make_partials(gen, S, B, H, D, empty_splits=()):
    po, pl = randn(gen, S, B, H, 1, D), torch.rand(S, B, H, 1, generator=gen) + 0.5
    pm = 3 * randn(gen, S, B, H, 1)
    for s in empty_splits:           # a split that saw no key (fa2.py: m = -inf, l = 0, acc = 0)
        po[s], pl[s], pm[s] = 0.0, 0.0, float("-inf")
    return po, pl, pm


@pytest.mark.parametrize("world,rank", [(1, 0), (2, 0), (2, 1), (4, 2)])
@pytest.mark.parametrize("o_dtype", [torch.float32, torch.bfloat16])
def test_merge_with_peers_played_by_the_test(cuda, world, rank, o_dtype):
    gen = torch.Generator().manual_seed(40 + world + rank)
    S, B, H, D = 6, 2, 4, 256
    rows, slices = B * H, D // COLS
    parts = [make_partials(gen, S, B, H, D, empty_splits=(1,) if r == 0 else ()) for r in range(world)]
    merged = [merged_partial(*p) for p in parts]
    want = orc.combine_partials(torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts]),
                                torch.cat([p[2] for p in parts]), world * S)

    peers = new_buffers(cuda, world, rows, slices)
    ex = PartialExchange(rows, D, peers=peers, rank=rank)
    # two launches: the launch count and the buffer parity advance on the device
    for epoch in (1, 2):
        par = epoch & 1
        for r in range(world):
            if r != rank:
                deliver(peers[rank], world, rows, slices, par, r, merged[r], epoch, cuda)
        o = torch.zeros(B, H, 1, D, dtype=o_dtype, device=cuda)
        po, pl, pm = (x.to(cuda) for x in parts[rank])
        ex.combine(po, pl, pm, o, S)
        tol = 1e-5 if o_dtype == torch.float32 else 8e-3
        assert torch.allclose(o.float().cpu(), want, atol=tol, rtol=tol), (o.float().cpu() - want).abs().max()
        # what this rank pushed to every rank: its merged partial, every word with the count
        acc, l, m = merged[rank]
        for r in range(world):
            w = words(peers[r], world, rows, slices)[par, rank].cpu()
            got = w[..., 0].contiguous().view(torch.float32)
            assert torch.allclose(got[..., :COLS].reshape(rows, D), acc.reshape(rows, D), atol=1e-5, rtol=1e-5)
            assert torch.allclose(got[..., COLS], l.reshape(rows, 1).expand(rows, slices), atol=1e-5, rtol=1e-5)
            assert torch.equal(got[..., COLS + 1], m.reshape(rows, 1).expand(rows, slices))
            assert (w[..., 1] == epoch).all()
        assert ex.state.tolist() == [epoch, 0]


def test_strided_packed_partials_and_phase_skip(cuda):
    """Partials as views of one packed [S,B,H,1,D+2] buffer (what the decode kernel writes into),
    and a slot off phase: its row of o keeps its content."""
    gen = torch.Generator().manual_seed(7)
    S, B, H, D = 16, 2, 8, 256
    po, pl, pm = make_partials(gen, S, B, H, D)
    packed = torch.cat([po, pl[..., None], pm[..., None]], -1).to(cuda)
    want = orc.combine_partials(po, pl, pm, S)
    rows, slices = B * H, D // COLS
    ex = PartialExchange(rows, D, peers=new_buffers(cuda, 1, rows, slices), rank=0)
    o = torch.full((B, H, 1, D), 7.0, device=cuda)
    phase = torch.tensor([2, 1], dtype=torch.uint8, device=cuda)
    ex.combine(packed[..., :D], packed[..., D], packed[..., D + 1], o, S, user_phase=phase, phase=2)
    assert torch.allclose(o[0].cpu(), want[0], atol=1e-5, rtol=1e-5)
    assert (o[1] == 7.0).all()


def test_bad_arguments_raise(cuda):
    peers = [torch.zeros(16, dtype=torch.int64, device=cuda)]
    with pytest.raises(ValueError):
        PartialExchange(8, 256, peers=peers, rank=0)        # buffers too small


def test_absent_peer_ends_in_a_status_code_not_a_hang(cuda):
    """A peer that never delivers: the bounded wait (about a second) runs out, the kernel
    returns, the status word names the wait, o is left alone and the context stays usable."""
    from g4b_b200 import _cabi

    gen = torch.Generator().manual_seed(3)
    S, B, H, D, world = 4, 1, 2, 256, 2
    rows, slices = B * H, D // COLS
    po, pl, pm = make_partials(gen, S, B, H, D)
    peers = new_buffers(cuda, world, rows, slices)
    ex = PartialExchange(rows, D, peers=peers, rank=0)
    o = torch.full((B, H, 1, D), 5.0, device=cuda)
    ex.combine(po.to(cuda), pl.to(cuda), pm.to(cuda), o, S)     # nothing ever writes rank 1's words
    assert _cabi.device_status() == 0x401                      # synchronises, reads and clears
    assert (o == 5.0).all()
    assert ex.state.tolist() == [1, 0]                          # the launch still completed its bookkeeping
    # the same object works again once the peer's pieces are there
    deliver(peers[0], world, rows, slices, 0, 1, merged_partial(po, pl, pm), 2, cuda)
    ex.combine(po.to(cuda), pl.to(cuda), pm.to(cuda), o, S)
    want = orc.combine_partials(torch.cat([po, po]), torch.cat([pl, pl]), torch.cat([pm, pm]), 2 * S)
    assert torch.allclose(o.cpu(), want, atol=1e-5, rtol=1e-5)
    assert _cabi.device_status() == 0
