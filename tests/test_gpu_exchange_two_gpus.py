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
