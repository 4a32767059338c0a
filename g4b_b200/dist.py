"""Multi-GPU partitioning of the attention path: one process per GPU.

The reference is single-GPU (one ``Device(0)``, g4b/__main__.py:46); everything here is new.
Three of the four sharded workloads need no communication at all (requests, kv heads and
sequences are independent).  Only single-sequence long-context decode exchanges data: every
rank attends to its contiguous share of the KV pages, and the per-rank (acc, l, m) partials --
the reference's split-KV format (g4b/kernels/fa2.py:438-472) -- are merged across ranks
(fa2.py:546-631 arithmetic).  Two forms: ``PartialExchange`` does it in one kernel over
peer-mapped memory; ``gather_packed`` + ``fa2.combine_partials`` all-gathers the partials with
the process group's backend (NCCL on GPUs, gloo on CPU tensors) and merges them with the same
kernel that merges intra-GPU splits.
"""
from __future__ import annotations

from typing import Sequence


def shard_requests(num_requests: int, world_size: int, rank: int) -> range:
    """Contiguous, balanced share of independent requests for ``rank``."""
    base, extra = divmod(num_requests, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def shard_request_heads(num_requests: int, kv_heads: int, world_size: int, rank: int) -> list[tuple[int, int]]:
    """(request, kv head) units of ``rank`` when there are more GPUs than requests: units are
    independent because a query head only reads its own kv head."""
    units = [(r, g) for r in range(num_requests) for g in range(kv_heads)]
    return [units[i] for i in shard_requests(len(units), world_size, rank)]


def shard_prefill_units(num_requests: int, kv_heads: int, seq_len: int, world_size: int, rank: int,
                        window: int | None = None) -> list[tuple[int, int, int, int, int]]:
    """Units of a prefill batch for ``rank``: (request, kv head, q_lo, q_hi, k_lo).

    A (request, kv head) pair is independent of every other (its query heads read only that kv
    head).  With more GPUs than pairs and a sliding window, the query range of every pair is
    also cut into equal parts: queries [q_lo, q_hi) then need the keys [k_lo, q_hi) with
    k_lo = max(0, q_lo - (window - 1)), a halo of window - 1 keys before the part.  Without a
    window a later part would need every earlier key and most of the work, so the query range
    is only cut for windowed attention.
    """
    pairs = [(r, g) for r in range(num_requests) for g in range(kv_heads)]
    parts = 1
    if window is not None and world_size > len(pairs):
        parts = world_size // len(pairs)
        while parts > 1 and seq_len % parts != 0:
            parts -= 1
    step = seq_len // parts
    units = []
    for r, g in pairs:
        for i in range(parts):
            q_lo, q_hi = i * step, (i + 1) * step
            units.append((r, g, q_lo, q_hi, max(0, q_lo - (window - 1)) if window is not None else 0))
    return [units[i] for i in shard_requests(len(units), world_size, rank)]


def balance_sequences(context_lens: Sequence[int], world_size: int) -> list[list[int]]:
    """Greedy longest-first assignment of sequences to GPUs so that KV bytes (proportional to
    context length) balance.  Returns the sequence indices of every rank."""
    order = sorted(range(len(context_lens)), key=lambda i: -int(context_lens[i]))
    loads = [0] * world_size
    out: list[list[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (loads[j], j))
        out[r].append(i)
        loads[r] += int(context_lens[i])
    for part in out:
        part.sort()
    return out


def split_pages(num_pages: int, world_size: int, rank: int) -> range:
    """Contiguous page range of ``rank`` for one long sequence split across GPUs."""
    return shard_requests(num_pages, world_size, rank)


def gather_partials(local_o, local_l, local_m, group=None):
    """All-gathers one (acc, l, m) partial per rank into split-major buffers.

    local_o [B,H,Tq,D], local_l / local_m [B,H,Tq] (f32; m in log2 units; acc un-normalised)
    -> partial_o [W,B,H,Tq,D], partial_l / partial_m [W,B,H,Tq], identical on every rank and
    ready for ``g4b_b200.kernels.fa2.combine_partials``.  Works on any torch.distributed
    backend (NCCL on GPUs, gloo on CPU tensors).
    """
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    po = torch.empty((world, *local_o.shape), dtype=local_o.dtype, device=local_o.device)
    pl = torch.empty((world, *local_l.shape), dtype=local_l.dtype, device=local_l.device)
    pm = torch.empty((world, *local_m.shape), dtype=local_m.dtype, device=local_m.device)
    # inputs get a leading split dim of 1 so the output is their concatenation along dim 0
    # (the only form every backend accepts)
    dist.all_gather_into_tensor(po, local_o.contiguous().unsqueeze(0), group=group)
    dist.all_gather_into_tensor(pl, local_l.contiguous().unsqueeze(0), group=group)
    dist.all_gather_into_tensor(pm, local_m.contiguous().unsqueeze(0), group=group)
    return po, pl, pm


def pack_partial(o, l, m):
    """One message instead of three: [...,D+2] = (acc | l | m)."""
    import torch

    return torch.cat([o, l.unsqueeze(-1), m.unsqueeze(-1)], dim=-1).contiguous()


def gather_packed(packed, out=None, group=None):
    """All-gather of packed partials [S,B,H,Tq,D+2] -> [W*S,B,H,Tq,D+2] (rank-major, i.e. the
    concatenation along the split dim); ``out`` may be preallocated."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty((world * packed.shape[0], *packed.shape[1:]), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(out, packed, group=group)
    return out


def unpack_gathered(gathered):
    """[S,B,H,Tq,D+2] -> strided views (partial_o, partial_l, partial_m) for the combine kernel."""
    d = gathered.shape[-1] - 2
    return gathered[..., :d], gathered[..., d], gathered[..., d + 1]


class PartialExchange:
    """Cross-GPU split-KV merge in one launch (``g4b_attn_combine_exchange``): the local
    partials are merged, the merged partials travel between the GPUs by plain stores into
    peer-mapped buffers as 8-byte words that carry the launch count beside the value (a word
    announces itself: no fence, no flag), and every rank finishes the merge -- no collective
    call, no second launch.

    ``PartialExchange(rows, head_dim)`` inside an initialised NCCL process group allocates the
    exchange buffer in symmetric memory (``torch.distributed._symmetric_memory``) and maps
    every peer's.  ``peers=[xbuf, ...]`` instead takes ready-made zeroed local tensors, one per
    rank (a world of one, or a test that plays the other ranks' part)."""

    def __init__(self, rows: int, head_dim: int, *, device=None, group=None, peers=None, rank=None):
        import torch

        from g4b_b200 import _cabi

        self._keep = []
        if peers is not None:
            self.world, self.rank = len(peers), int(rank or 0)
        else:
            import torch.distributed as dist

            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.xbuf_bytes = int(_cabi.load().g4b_exchange_buffer_bytes(self.world, rows, head_dim))
        if peers is not None:
            self.xbuf_ptrs = [int(x.data_ptr()) for x in peers]
            for x in peers:
                if x.numel() * x.element_size() < self.xbuf_bytes:
                    raise ValueError(f"exchange buffers need {self.xbuf_bytes} bytes per rank")
            self._keep += list(peers)
            device = peers[self.rank].device
        else:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm

            device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
            name = (group or dist.group.WORLD).group_name
            xbuf = symm.empty(self.xbuf_bytes // 8, dtype=torch.int64, device=device)
            xbuf.zero_()
            hx = symm.rendezvous(xbuf, name)
            self.xbuf_ptrs = [int(p) for p in hx.buffer_ptrs]
            self._keep += [xbuf, hx]
            torch.cuda.synchronize(device)
            dist.barrier(group)      # nobody pushes before every rank's buffer is zero
        self.state = torch.zeros(2, dtype=torch.int32, device=device)

    def combine(self, partial_o, partial_l, partial_m, o, num_splits: int, *, user_phase=None, phase: int = 2, stream=None):
        """Merges this rank's first ``num_splits`` partials with every other rank's into ``o``.
        All ranks must call it the same number of times with the same shapes."""
        import ctypes

        from g4b_b200 import _cabi

        a = _cabi.G4bExchangeArgs()
        a.partial_o = _cabi.as_tensor(partial_o)
        a.partial_l = _cabi.as_tensor(partial_l)
        a.partial_m = _cabi.as_tensor(partial_m)
        a.o = _cabi.as_tensor(o)
        a.user_phase = _cabi.as_tensor(user_phase)
        for r in range(self.world):
            a.xbuf[r] = self.xbuf_ptrs[r]
        a.state = self.state.data_ptr()
        a.xbuf_bytes = self.xbuf_bytes
        a.num_splits, a.phase, a.world, a.rank = int(num_splits), int(phase), self.world, self.rank
        _cabi.check(_cabi.load().g4b_attn_combine_exchange(ctypes.byref(a), ctypes.c_void_p(_cabi.current_stream(stream))))
        return None
