"""The cross-GPU split-KV merge over real peer memory: two processes, one GPU each, NCCL for
the rendezvous only, the exchange kernel for the data.  Needs two GPUs in the machine (skipped
otherwise; the one-GPU tests play the peers' part themselves).  Every rank knows every rank's
partials (same seeds), so each checks its own output against the oracle's merge of all of them.
Nothing here can wait for ever: the kernel's waits run out after about a second and leave a
status code, and the parent gives the children two minutes."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

S, B, H, D, STEPS = 12, 2, 8, 256, 4


def _partials(rank, step):
    gen = torch.Generator().manual_seed(1000 + 17 * rank + step)
    po = torch.randn(S, B, H, 1, D, generator=gen)
    pl = torch.rand(S, B, H, 1, generator=gen) + 0.5
    pm = 3 * torch.randn(S, B, H, 1, generator=gen)
    if rank == 0:                      # a split that saw no key (fa2.py: m = -inf, l = 0, acc = 0)
        po[1], pl[1], pm[1] = 0.0, 0.0, float("-inf")
    return po, pl, pm


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from g4b_b200 import _cabi
    from g4b_b200.dist import PartialExchange
    from helpers import orc

    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        ex = PartialExchange(B * H, D, device=dev)
        worst = 0.0
        for step in range(STEPS):      # several launches: the buffer parity and the launch count advance
            parts = [_partials(r, step) for r in range(world)]
            want = orc.combine_partials(torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts]),
                                        torch.cat([p[2] for p in parts]), world * S)
            po, pl, pm = (x.to(dev) for x in parts[rank])
            o = torch.zeros(B, H, 1, D, device=dev)
            ex.combine(po, pl, pm, o, S)
            worst = max(worst, float((o.cpu() - want).abs().max()))
        status = _cabi.device_status()
        results.put((rank, worst, status, ex.state.tolist()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_exchange_between_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29400 + os.getpid() % 500
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:
        p.terminate()
    assert not stuck, "a rank did not finish"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    got = sorted(results.get(timeout=5) for _ in range(2))
    for rank, worst, status, state in got:
        assert status == 0, f"rank {rank}: device status {status:#x}"
        assert worst < 1e-5, f"rank {rank}: max error {worst}"
        assert state == [STEPS, 0]


def _step_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from g4b_b200 import _cabi
    from g4b_b200.dist import PartialExchange, split_pages
    from g4b_b200.kernels import fa2
    from helpers import orc, randn

    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        Hq, G, Dh, L, Sp = 8, 2, 256, 16 * 90, 5
        gen = torch.Generator().manual_seed(77)                   # the same sequence on every rank
        k, v = randn(gen, G, L, Dh, dtype=torch.bfloat16), randn(gen, G, L, Dh, dtype=torch.bfloat16)
        rng = split_pages(L // 16, world, rank)
        lo, n = rng.start * 16, len(rng)
        kp = k[:, lo:lo + 16 * n].reshape(G, n, 16, Dh).permute(1, 0, 2, 3).contiguous().to(dev)
        vp = v[:, lo:lo + 16 * n].reshape(G, n, 16, Dh).permute(1, 0, 2, 3).contiguous().to(dev)
        bt = torch.arange(n, dtype=torch.int32, device=dev)[None]
        time = torch.tensor([16 * n], dtype=torch.int32, device=dev)
        ex = PartialExchange(Hq, Dh, device=dev)
        po, pl, pm = (torch.empty(Sp, 1, Hq, 1, Dh, device=dev), torch.empty(Sp, 1, Hq, 1, device=dev),
                      torch.empty(Sp, 1, Hq, 1, device=dev))
        worst = -1.0
        for step in range(STEPS):
            q = randn(gen, 1, Hq, 1, Dh, dtype=torch.bfloat16)
            want = orc.attention_core(q[0], k, v, scale=1 / 16)[None]
            o = torch.zeros(1, Hq, 1, Dh, dtype=torch.bfloat16, device=dev)
            fa2.decode_step(q.to(dev), kp, vp, o, time, None, 16 * n, fa2.PHASE_DECODE, po, pl, pm, exchange=ex,
                            num_kv_splits=Sp, scale=1 / 16, block_tables=bt, page_size=16)
            err = (o.float().cpu() - want).abs() - (2e-3 + 1e-2 * want.abs())
            worst = max(worst, float(err.max()))
        status = _cabi.device_status()
        results.put((rank, worst, status, int(ex.state[0])))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_decode_step_exchange_between_two_gpus():
    """One sequence split over two real GPUs, g4b_decode_step with peers: every rank's output
    against the oracle's attention over the whole sequence, four steps in a row."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29900 + os.getpid() % 90
    procs = [ctx.Process(target=_step_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:
        p.terminate()
    assert not stuck, "a rank did not finish"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for rank, worst, status, launches in sorted(results.get(timeout=5) for _ in range(2)):
        assert status == 0, f"rank {rank}: device status {status:#x}"
        assert worst <= 0, f"rank {rank}: tolerance exceeded by {worst}"
        assert launches == STEPS
