"""Host-side multi-GPU logic on CPU: partitioning helpers, and the cross-rank split-KV
exchange run as two gloo ranks (the (acc, l, m) partials of two halves of one sequence are
all-gathered and merged; the result must equal unsplit attention)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from g4b_b200 import dist as gdist
from helpers import orc


def test_shard_requests_cover_and_balance():
    for n in (1, 4, 7, 256):
        for w in (1, 2, 4, 8):
            parts = [list(gdist.shard_requests(n, w, r)) for r in range(w)]
            assert sorted(sum(parts, [])) == list(range(n))
            sizes = [len(p) for p in parts]
            assert max(sizes) - min(sizes) <= 1


def test_shard_request_heads_for_more_gpus_than_requests():
    units = [gdist.shard_request_heads(4, 2, 8, r) for r in range(8)]
    assert all(len(u) == 1 for u in units)
    assert sorted(sum(units, [])) == [(r, g) for r in range(4) for g in range(2)]


def test_shard_prefill_units_cover_every_query_once():
    # config 2 (4 requests, causal) and config 3 (2 requests, window 512) at 1, 2, 4 and 8 GPUs
    for n_req, S, W in ((4, 8192, None), (2, 32768, 512)):
        for w in (1, 2, 4, 8):
            units = sum((gdist.shard_prefill_units(n_req, 2, S, w, r, W) for r in range(w)), [])
            per_rank = [len(gdist.shard_prefill_units(n_req, 2, S, w, r, W)) for r in range(w)]
            assert max(per_rank) - min(per_rank) <= (0 if len(units) % w == 0 else 1)
            seen = {}
            for r, g, q_lo, q_hi, k_lo in units:
                assert 0 <= k_lo <= q_lo < q_hi <= S
                assert k_lo == (max(0, q_lo - (W - 1)) if W else 0)
                seen.setdefault((r, g), []).append((q_lo, q_hi))
            assert sorted(seen) == [(r, g) for r in range(n_req) for g in range(2)]
            for rngs in seen.values():
                rngs.sort()
                assert rngs[0][0] == 0 and rngs[-1][1] == S
                assert all(a[1] == b[0] for a, b in zip(rngs, rngs[1:]))
    # the query range is cut only when there are more GPUs than pairs and a window
    assert len(gdist.shard_prefill_units(2, 2, 32768, 8, 0, 512)) == 1
    assert gdist.shard_prefill_units(2, 2, 32768, 8, 1, 512)[0] == (0, 0, 16384, 32768, 16384 - 511)
    assert len(gdist.shard_prefill_units(4, 2, 8192, 8, 3, None)) == 1


def test_balance_sequences_longest_first():
    gen = torch.Generator().manual_seed(0)
    lens = torch.randint(1024, 32769, (256,), generator=gen).tolist()
    for w in (2, 4, 8):
        parts = gdist.balance_sequences(lens, w)
        assert sorted(sum(parts, [])) == list(range(256))
        loads = [sum(lens[i] for i in p) for p in parts]
        assert (max(loads) - min(loads)) / (sum(loads) / w) < 0.01


def test_split_pages_contiguous():
    for w in (1, 2, 4, 8):
        rngs = [gdist.split_pages(8192, w, r) for r in range(w)]
        assert rngs[0].start == 0 and rngs[-1].stop == 8192
        assert all(a.stop == b.start for a, b in zip(rngs, rngs[1:]))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q, k, v, local_splits, result_dict):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world)
    try:
        Tk = k.shape[1]
        n_pages = (Tk + 15) // 16
        rng = gdist.split_pages(n_pages, world, rank)
        lo, hi = rng.start * 16, min(Tk, rng.stop * 16)
        acc, l, m = orc.split_partials(q, k[:, lo:hi], v[:, lo:hi], scale=1 / 16, num_splits=local_splits)
        # [S,H,1,D] -> [S,B=1,H,1,D]; one packed message per rank
        packed = gdist.pack_partial(acc[:, None], l[:, None], m[:, None])
        gathered = gdist.gather_packed(packed)
        assert gathered.shape == (world * local_splits, 1, q.shape[0], 1, q.shape[2] + 2)
        go, gl, gm = gdist.unpack_gathered(gathered)
        out = orc.combine_partials(go, gl, gm, world * local_splits)
        # the three-tensor form must agree with the packed form
        po, pl, pm = gdist.gather_partials(acc[0][None], l[0][None], m[0][None])
        assert torch.equal(po[rank], acc[0][None]) and po.shape[0] == world
        result_dict[rank] = out[0]
    finally:
        torch.distributed.destroy_process_group()


@pytest.mark.timeout(120)
def test_cross_rank_split_kv_exchange_gloo():
    gen = torch.Generator().manual_seed(11)
    H, G, D, Tk = 8, 2, 64, 1000
    q = torch.randn(H, 1, D, generator=gen)
    k = torch.randn(G, Tk, D, generator=gen)
    v = torch.randn(G, Tk, D, generator=gen)
    want = orc.attention_core(q, k, v, scale=1 / 16)
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_rank_main, args=(world, port, q, k, v, 3, results), nprocs=world, join=True)
        assert len(results) == world
        for r in range(world):
            assert torch.allclose(results[r], want, atol=1e-5, rtol=1e-4), f"rank {r}"
        assert torch.equal(results[0], results[1])
