"""The whole path as a serving loop would drive it, on the GPU: host page manager -> block
tables, fused norm + rotary + append, paged attention (chunked prefill, then decode with the
state advanced on the device), for several requests that come and go and share prefixes.

Every step's attention output of every live slot is compared with the oracle run on that
request alone over contiguous K/V, so a wrong page, a stale shared page, a wrong position or
a missed upload all show.  Token 'embeddings' are seeded tables, so equal prefixes give
equal K/V, which is what makes page sharing checkable."""
import pytest
import torch

from g4b_b200.kernels.advance_decode_state import advance_decode_state
from g4b_b200.kernels.fa2 import flash_attention
from g4b_b200.kernels.rope import rope_norm_append
from g4b_b200.paging import PagedKVManager
from helpers import assert_close, orc

pytestmark = pytest.mark.gpu

H, G, D, PAGE, CHUNK, VOCAB, B = 4, 2, 256, 16, 32, 50, 3
SCALE = 1 / 16


class Tables:
    def __init__(self, device):
        gen = torch.Generator().manual_seed(1234)
        self.q = torch.randn(VOCAB, H, D, generator=gen)
        self.k = torch.randn(VOCAB, G, D, generator=gen)
        self.v = torch.randn(VOCAB, G, D, generator=gen)
        self.q_w = 1 + 0.1 * torch.randn(D, generator=gen)
        self.k_w = 1 + 0.1 * torch.randn(D, generator=gen)
        self.freqs = 1.0 / (10000.0 ** (torch.arange(0, D, 2) / D))
        self.dev = {n: getattr(self, n).to(device) for n in ("q", "k", "v", "q_w", "k_w", "freqs")}


def oracle_rows(tab, tokens, first, count):
    """What the oracle puts into the cache and into q for one request alone: q of positions
    [first, first+count) and K/V of positions [0, first+count), fp32, all contiguous."""
    n = first + count
    ids = torch.tensor(tokens[:n])
    pos = torch.arange(n)[None]
    q = orc.rope_norm(tab.q[ids].permute(1, 0, 2)[None], pos, tab.freqs, weight=tab.q_w)
    k = orc.rope_norm(tab.k[ids].permute(1, 0, 2)[None], pos, tab.freqs, weight=tab.k_w)
    v = orc.rope_norm(tab.v[ids].permute(1, 0, 2)[None], pos, None)
    return q[0][:, first:], k[0], v[0]


def one_bf16_ulp(got, want):
    """got (bf16 values as fp32) equals want rounded to bf16, or its neighbour: the norm's
    rsqrt and the rotation's sine and cosine are approximations on both sides, so a value that
    sits on a rounding boundary may fall either way."""
    return bool(((got - want).abs() <= want.abs() * 2.0 ** -7 + 1e-6).all())


def check_step(tab, tokens, first, count, q16_slot, o_slot, k_pool, v_pool, table_row, what):
    """(1) The rows the GPU holds for this request -- the rotated q of the step and, read through
    the slot's block table, every K/V row of the context -- are the oracle's rows within one
    bf16 rounding: a wrong page, a stale shared page or a wrong position shows here.  (2) The
    attention output equals the oracle's attention over exactly those GPU-held rows at the
    tolerance of every other parity test."""
    n = first + count
    q_want, k_want, v_want = oracle_rows(tab, tokens, first, count)
    pages = torch.as_tensor(table_row[: (n + PAGE - 1) // PAGE]).long().to(k_pool.device)
    k_gpu = k_pool[pages].float().cpu().permute(1, 0, 2, 3).reshape(G, -1, D)[:, :n]
    v_gpu = v_pool[pages].float().cpu().permute(1, 0, 2, 3).reshape(G, -1, D)[:, :n]
    q_gpu = q16_slot[:, :count].float().cpu()
    assert one_bf16_ulp(k_gpu, k_want), f"{what}: K rows in the pages differ from the oracle's"
    assert one_bf16_ulp(v_gpu, v_want), f"{what}: V rows in the pages differ from the oracle's"
    assert one_bf16_ulp(q_gpu, q_want), f"{what}: rotated q differs from the oracle's"
    want = orc.attention_core(q_gpu, k_gpu, v_gpu, scale=SCALE, causal=True)
    assert_close(o_slot[:, :count], want, what)


def next_token(tok):
    return (tok * 7 + 3) % VOCAB


def test_requests_come_and_go_over_shared_pages(cuda):
    tab = Tables(cuda)
    mgr = PagedKVManager(num_pages=40, max_batch=B, max_context=256, page_size=PAGE, prefill_chunk=CHUNK,
                         decode_reserve_pages=1)
    mgr.bind_device(cuda)
    k_pool = torch.zeros(40, G, PAGE, D, dtype=torch.bfloat16, device=cuda)
    v_pool = torch.zeros_like(k_pool)
    cw = mgr.max_pages * PAGE
    gen = torch.Generator().manual_seed(5)
    base = torch.randint(0, VOCAB, (120,), generator=gen).tolist()
    prompts = [base[:70], base[:66] + [1, 2, 3, 4, 5, 6], torch.randint(0, VOCAB, (80,), generator=gen).tolist(),
               base[:100]]
    n_decode = [20, 5, 9, 4]
    arrival = [0, 2, 0, 30]       # loop iteration at which each request shows up

    class Rq:
        def __init__(self, idx):
            self.idx, self.tokens, self.slot, self.pos, self.left = idx, list(prompts[idx]), None, 0, n_decode[idx]

    waiting = [Rq(i) for i in range(len(prompts))]
    active: list[Rq | None] = [None] * B
    shared_tokens = 0
    checked = 0

    def run_step(phase, t, ids_dev, dev):
        """One model step for all slots: gather embeddings, fused rotary/append, attention."""
        q = tab.dev["q"][ids_dev].permute(0, 2, 1, 3)             # [B,t,H,D] physical, [B,H,t,D] view
        k = tab.dev["k"][ids_dev].permute(0, 2, 1, 3)
        v = tab.dev["v"][ids_dev].permute(0, 2, 1, 3)
        q16 = torch.zeros(B, H, t, D, dtype=torch.bfloat16, device=cuda)
        o = torch.zeros(B, H, t, D, dtype=torch.bfloat16, device=cuda)
        rope_norm_append(q, k, v, tab.dev["freqs"], dev["cache_offsets"], k_pool, v_pool, 1e-6, q_out=q16,
                         q_rmsnorm_w=tab.dev["q_w"], k_rmsnorm_w=tab.dev["k_w"], user_phase=dev["user_phase"],
                         phase=phase, block_tables=dev["block_tables"], page_size=PAGE)
        flash_attention(q16, k_pool, v_pool, o, dev["time_dim_sizes"], dev["user_phase"], cw, phase, scale=SCALE,
                        block_tables=dev["block_tables"], page_size=PAGE)
        return o, q16

    in_ids = torch.zeros(1, B, dtype=torch.int32, device=cuda)    # decode feedback buffers
    out_ids = torch.zeros(B, 1, dtype=torch.int32, device=cuda)
    decode_uploaded = False
    for it in range(300):
        # admission, as the reference does it: only while nobody is decoding (scheduler.py:97-98)
        if not any(r is not None and r.pos >= len(prompts[r.idx]) for r in active):
            while waiting and None in active and (arrival[waiting[0].idx] <= it or all(x is None for x in active)):
                r = waiting.pop(0)
                r.slot, r.pos = mgr.place_request(r.tokens)
                shared_tokens += r.pos
                active[r.slot] = r
        live = [r for r in active if r is not None]
        if not live:
            break
        # decode has priority over prefill (scheduler.py:66)
        if not any(r.pos >= len(prompts[r.idx]) for r in live):
            # ---- prefill step: chunk of CHUNK tokens per slot that still has prompt left
            off, tim = [0] * B, [0] * B
            ids = torch.zeros(B, CHUNK, dtype=torch.long)
            todo = []
            for r in live:
                n_prompt = len(prompts[r.idx])
                if r.pos >= n_prompt:
                    continue
                end = min(r.pos + CHUNK, n_prompt)
                toks = r.tokens[r.pos:end]
                ids[r.slot] = torch.tensor(toks + [toks[-1]] * (CHUNK - len(toks)))
                off[r.slot], tim[r.slot] = r.pos, r.pos + CHUNK            # padded chunk counts (scheduler.py:166-172)
                todo.append((r, r.pos, end - r.pos))
                r.pos = end
            mgr.prepare_prefill_inputs(None, off, tim)
            dev = mgr.upload()
            o, q16 = run_step(1, CHUNK, ids.to(cuda), dev)
            for r, first, count in todo:
                check_step(tab, r.tokens, first, count, q16[r.slot], o[r.slot], k_pool, v_pool,
                           mgr.block_tables[r.slot], f"prefill rq{r.idx} at {first}")
                checked += 1
                if r.pos >= len(prompts[r.idx]):
                    r.tokens.append(next_token(r.tokens[-1]))             # 'sampled' from the last prompt token
            decode_uploaded = False
            continue
        # ---- decode step: slots still in prefill sit it out
        live = [r for r in live if r.pos >= len(prompts[r.idx])]
        if not decode_uploaded:
            off, tim = [0] * B, [0] * B
            host_ids = [0] * B
            for r in live:
                off[r.slot], tim[r.slot] = len(r.tokens) - 1, len(r.tokens)   # scheduler.py:199-203
                host_ids[r.slot] = r.tokens[-1]
            mgr.prepare_decode_inputs(None, off, tim)
            dev = mgr.upload()
            in_ids.copy_(torch.tensor([host_ids], dtype=torch.int32))
            decode_uploaded = True
        o, q16 = run_step(2, 1, in_ids[0].long()[:, None], dev)
        for r in live:
            check_step(tab, r.tokens, len(r.tokens) - 1, 1, q16[r.slot], o[r.slot], k_pool, v_pool,
                       mgr.block_tables[r.slot], f"decode rq{r.idx} at {len(r.tokens) - 1}")
            checked += 1
        # the sampler's stand-in writes the next token; the state advances on the device
        nxt = [0] * B
        for r in live:
            nxt[r.slot] = next_token(r.tokens[-1])
        out_ids.copy_(torch.tensor(nxt, dtype=torch.int32)[:, None])
        advance_decode_state(in_ids, out_ids, dev["cache_offsets"], dev["time_dim_sizes"], dev["user_phase"])
        if mgr.advance_decode():
            mgr.upload()                                                  # new pages: tables change, state is equal
        for r in list(live):
            r.tokens.append(nxt[r.slot])
            r.left -= 1
            if r.left == 0:
                mgr.retire(r.slot, r.tokens[:-1])
                active[r.slot] = None
                decode_uploaded = False
        assert torch.equal(dev["time_dim_sizes"].cpu(), torch.from_numpy(mgr.time_dim_sizes)), "host mirror drifted"
    assert not waiting and all(r is None for r in active)
    # rq1 shares 32 tokens with rq0 while rq0 is still running; rq3 reuses rq0's retired slot (64)
    assert shared_tokens == 32 + 64, shared_tokens
    assert checked > 40
