"""CPU oracle for the attention hot path -- TEST INFRASTRUCTURE, not the product.

A restatement, in plain torch fp32 / numpy on the CPU, of what the reference computes on
this path.  Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
it; the product (g4b_b200) never does and has no CPU fallback.

Parity status: PINNED.  tests/test_oracle_golden.py checks every function here against
outputs of the reference's own torch implementation (scripts/reference_impl.py,
LayerKVCache.add / .retrieve), generated in the build container by
tests/golden/make_golden.py and committed as tests/golden/*.npz.  The reference's own tests
for this path hold no golden vectors or assertions (tests/compare_scripts/test_fa2.py and
test_add_kv.py only print differences).

What each function follows:
  attention_core        scripts/reference_impl.py:434-443  (LayerKVCache.retrieve)
  unroll_ring           g4b/kernels/fa2.py:52-55,75; tests/compare_scripts/test_fa2.py:128-132
  gather_pages          new (paged layout): pool[block_table[j // page], :, j % page, :]
  flash_attention       g4b/kernels/fa2.py:256-480 semantics over the above
  add_kv_to_cache       g4b/kernels/add_kv_to_cache.py:148-158
  rope_norm             g4b/kernels/rope.py:22-39,166-173; scripts/reference_impl.py:77-85,255-265
  rope_norm_append      the sequence at g4b/models/gemma4e.py:564-592 over the two above
  advance_decode_state  g4b/kernels/advance_decode_state.py:52-63
  combine_partials      g4b/kernels/fa2.py:618-626
  select_kv_splits      g4b/kernels/fa2.py:201-212
  add_kv_to_cache_fp8   new (8-bit cache): the append of add_kv_to_cache.py:148-158 followed by the
                        quantiser stated in include/g4b_attn.h (scale of a page from its first row)
  dequantise_fp8_pool   new: e4m3(byte) x scale; attention over an 8-bit pool is the attention
                        above over these values
"""
from __future__ import annotations

import math

import numpy as np
import torch

PHASE_UNALLOCATED, PHASE_PREFILL, PHASE_DECODE = 0, 1, 2
STAGE_FULL, STAGE_CAUSAL = 1, 3


def attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float = 1.0,
                   causal: bool = True, sliding_window: int | None = None,
                   q_block: int = 1024) -> torch.Tensor:
    """softmax(scale * q k^T + mask) v in fp32 for one sequence.

    q [H,Tq,D], k/v [G,Tk,D]; the queries are the LAST Tq positions of the Tk keys
    (reference_impl.py:437-438: q_pos = arange(t_end - Tq, t_end), k_pos = arange(t_start,
    t_end)).  Masked where q_pos < k_pos (:439) and, with a sliding window W, where
    q_pos - k_pos >= W (:440-441).  GQA by repeat_interleave (:434-435).  The reference is
    unscaled (:443); ``scale`` multiplies q first, in fp32.  Rows with no visible key give 0.
    Evaluated in blocks of ``q_block`` queries to bound memory; the arithmetic per row is the
    reference's.
    """
    q = q.to(torch.float32) * float(scale)
    k = k.to(torch.float32)
    v = v.to(torch.float32)
    H, Tq, D = q.shape
    G, Tk, _ = k.shape
    rep = H // G
    kk = torch.repeat_interleave(k, rep, 0)
    vv = torch.repeat_interleave(v, rep, 0)
    out = torch.empty(H, Tq, v.shape[-1], dtype=torch.float32)
    k_pos = torch.arange(0, Tk)[None, :]
    for s in range(0, Tq, q_block):
        e = min(Tq, s + q_block)
        q_pos = torch.arange(Tk - Tq + s, Tk - Tq + e)[:, None]
        mask = torch.zeros(e - s, Tk, dtype=torch.bool)
        if causal:
            mask |= q_pos < k_pos
        if sliding_window is not None and sliding_window > 0:
            mask |= (q_pos - k_pos) >= sliding_window
        # only the key range any row of the block can see has to be multiplied
        vis = (~mask).any(0).nonzero()
        if vis.numel() == 0:
            out[:, s:e] = 0
            continue
        lo, hi = int(vis.min()), int(vis.max()) + 1
        scores = q[:, s:e] @ kk[:, lo:hi].transpose(-1, -2)
        scores = scores + torch.where(mask[:, lo:hi], float("-inf"), 0.0)
        dead = mask[:, lo:hi].all(-1)
        p = scores.softmax(-1)
        p = torch.where(dead[None, :, None], torch.zeros((), dtype=p.dtype), p)
        out[:, s:e] = p @ vv[:, lo:hi]
    return out


def unroll_ring(cache_b: torch.Tensor, time_dim_size: int, ctx_window_size: int) -> torch.Tensor:
    """Logical key order of one slot's ring buffer [G,T,D] -> [G,window,D]:
    window = min(time, ctx_window); ring_start = max(time - ctx_window, 0) % T; logical key j
    is row (ring_start + j) % T (fa2.py:52-55,75)."""
    T = cache_b.shape[1]
    window = min(int(time_dim_size), int(ctx_window_size))
    ring_start = max(int(time_dim_size) - int(ctx_window_size), 0) % T
    idx = (ring_start + torch.arange(window)) % T
    return cache_b[:, idx]


def gather_pages(pool: torch.Tensor, block_table_b: torch.Tensor, length: int, page_size: int) -> torch.Tensor:
    """Logical keys [0, length) of one sequence from a page pool [num_pages,G,page,D] -> [G,length,D]."""
    j = torch.arange(int(length))
    pages = block_table_b.to(torch.int64)[j // page_size]
    return pool[pages, :, j % page_size].permute(1, 0, 2)


def flash_attention(q, k_cache, v_cache, o, time_dim_sizes, user_phase, ctx_window_size, phase, *,
                    stage=STAGE_CAUSAL, scale=1.0, sliding_window=None, block_tables=None,
                    page_size=16) -> torch.Tensor:
    """Oracle of the whole op: returns a new fp32 ``o`` [B,H,Tq,D]; slots off-phase keep the
    values of the ``o`` passed in (fa2.py:333-335).

    Slot b sees its last ``window = min(time[b], ctx_window_size)`` keys (fa2.py:53) in
    logical order; its Tq queries are the last Tq of them (fa2.py:55-56), causal when
    ``stage`` is STAGE_CAUSAL (fa2.py:93-96).  ``sliding_window=None`` is the reference
    kernel's chunk-shared window (every query sees back to logical key 0, fa2.py:58-64);
    a value W adds the per-query bound of reference_impl.py:440-441.
    """
    B, H, Tq, D = q.shape
    out = o.detach().to(torch.float32).clone()
    for b in range(B):
        if user_phase is not None and int(user_phase[b]) != int(phase):
            continue
        time = int(time_dim_sizes[b])
        window = min(time, int(ctx_window_size))
        if block_tables is None:
            k = unroll_ring(k_cache[b], time, ctx_window_size)
            v = unroll_ring(v_cache[b], time, ctx_window_size)
        else:
            # paged caches hold absolute positions; the window is their tail
            k = gather_pages(k_cache, block_tables[b], time, page_size)[:, time - window:]
            v = gather_pages(v_cache, block_tables[b], time, page_size)[:, time - window:]
        if window == 0:
            out[b] = 0
            continue
        # queries are the last Tq logical positions; rows that precede every key give 0
        out[b] = attention_core(q[b], k, v, scale=scale, causal=(stage == STAGE_CAUSAL),
                                sliding_window=sliding_window)
    return out


def add_kv_to_cache(x, cache, cache_offsets, rmsnorm_eps, x_rsos=None, user_phase=None, phase=0, *,
                    block_tables=None, page_size=16) -> torch.Tensor:
    """Returns the cache after the append (a copy).  cache[b,g,(off[b]+t) % T,:] =
    cast(x[b,g,t,:] * r), r = rsqrt(rsos/D + eps) or 1 (add_kv_to_cache.py:148-158); paged:
    row off[b]+t of the sequence lands in page block_tables[b, p // page], row p % page."""
    out = cache.detach().clone()
    B, G, Tq, D = x.shape
    xf = x.detach().to(torch.float32)
    if x_rsos is not None:
        r = 1.0 / torch.sqrt(x_rsos.detach().to(torch.float32) / D + rmsnorm_eps)
        xf = xf * r[..., None]
    val = xf.to(cache.dtype) if (x_rsos is not None or x.dtype != cache.dtype) else x.detach()
    for b in range(B):
        if user_phase is not None and int(user_phase[b]) != int(phase):
            continue
        off = int(cache_offsets[b])
        for t in range(Tq):
            pos = off + t
            if block_tables is None:
                out[b, :, pos % cache.shape[2]] = val[b, :, t]
            else:
                page = int(block_tables[b, pos // page_size])
                out[page, :, pos % page_size] = val[b, :, t]
    return out


def rope_norm(x, positions, rope_freqs, *, rsos=None, weight=None, eps=1e-6, norm=True) -> torch.Tensor:
    """x [B,heads,t,D] -> fp32 rows scaled by rsqrt(rsos/D + eps) * weight (rsos defaults to the
    row's own sum of squares) and rotated: pairs (i, i + D/2) turn by theta =
    positions[b,t] * rope_freqs[i], theta an fp32 product (rope.py:22-39,166-173;
    reference_impl.py:259-265).  rope_freqs None = no rotation; norm False = no scaling."""
    xf = x.detach().to(torch.float32)
    D = xf.shape[-1]
    if norm:
        ss = xf.square().sum(-1) if rsos is None else rsos.detach().to(torch.float32)
        inv = torch.rsqrt(ss / D + eps)[..., None]
        xf = xf * (inv * weight.to(torch.float32) if weight is not None else inv)
    if rope_freqs is None:
        return xf
    theta = positions.to(torch.float32)[:, None, :, None] * rope_freqs.to(torch.float32)[None, None, None, :]
    sin, cos = theta.sin(), theta.cos()
    x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
    return torch.cat([cos * x1 - sin * x2, cos * x2 + sin * x1], dim=-1)


def rope_norm_append(q, k, v, rope_freqs, cache_offsets, k_cache, v_cache, rmsnorm_eps, *, q_rsos=None,
                     k_rsos=None, v_rsos=None, q_rmsnorm_w=None, k_rmsnorm_w=None, norm_qk=True, norm_v=True,
                     user_phase=None, phase=0, block_tables=None, page_size=16):
    """Returns (q', k', k_cache', v_cache'): q and k normalised and rotated in fp32 (not phase
    gated), and the caches after appending k' and the normalised v for the slots in phase
    (g4b/models/gemma4e.py:564-592)."""
    B, _, Tq, D = q.shape
    pos = cache_offsets.to(torch.int64)[:, None] + torch.arange(Tq)[None, :]
    q2 = rope_norm(q, pos, rope_freqs, rsos=q_rsos, weight=q_rmsnorm_w, eps=rmsnorm_eps, norm=norm_qk)
    k2 = rope_norm(k, pos, rope_freqs, rsos=k_rsos, weight=k_rmsnorm_w, eps=rmsnorm_eps, norm=norm_qk)
    kc = add_kv_to_cache(k2, k_cache, cache_offsets, rmsnorm_eps, None, user_phase, phase,
                         block_tables=block_tables, page_size=page_size) if k_cache is not None else None
    vc = None
    if v is not None:
        v2 = rope_norm(v, pos, None, rsos=v_rsos, eps=rmsnorm_eps, norm=norm_v)
        vc = add_kv_to_cache(v2, v_cache, cache_offsets, rmsnorm_eps, None, user_phase, phase,
                             block_tables=block_tables, page_size=page_size)
    return q2, k2, kc, vc


def advance_decode_state(input_token_ids, out_token_ids, cache_offsets, time_dim_sizes, user_phase):
    """Returns updated copies (input_token_ids, cache_offsets, time_dim_sizes) as numpy int32
    (advance_decode_state.py:52-63)."""
    inp = np.array(input_token_ids, dtype=np.int32, copy=True)
    off = np.array(cache_offsets, dtype=np.int32, copy=True)
    tim = np.array(time_dim_sizes, dtype=np.int32, copy=True)
    out_tok = np.asarray(out_token_ids)
    ph = np.asarray(user_phase)
    sel = ph == PHASE_DECODE
    inp[0, sel] = out_tok[sel, 0]
    off[sel] += 1
    tim[sel] += 1
    return inp, off, tim


def combine_partials(partial_o, partial_l, partial_m, num_splits) -> torch.Tensor:
    """o = (sum_s acc_s 2^(m_s - m)) / (sum_s l_s 2^(m_s - m)), m = max_s m_s, running form of
    fa2.py:618-626; m in log2 units.  partial_o [S,B,H,Tq,D], l/m [S,B,H,Tq] -> [B,H,Tq,D]."""
    po = partial_o[:num_splits].to(torch.float32)
    pl = partial_l[:num_splits].to(torch.float32)
    pm = partial_m[:num_splits].to(torch.float32)
    m = torch.full_like(pm[0], float("-inf"))
    l = torch.zeros_like(pl[0])
    acc = torch.zeros_like(po[0])
    for s in range(num_splits):
        m_new = torch.maximum(pm[s], m)
        safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
        a_new = torch.exp2(pm[s] - safe)
        a_cur = torch.exp2(m - safe)
        acc = acc * a_cur[..., None] + po[s] * a_new[..., None]
        l = l * a_cur + pl[s] * a_new
        m = m_new
    return acc / l[..., None]


def split_partials(q_b, k, v, *, scale: float, num_splits: int, block: int = 16):
    """Reference-format partials of ONE sequence for Tq == 1: un-normalised acc, l and m (log2
    units) per split (fa2.py:438-472), over contiguous ranges of ceil(nblocks/S) 16-key blocks.
    q_b [H,1,D], k/v [G,Tk,D] -> (acc [S,H,1,D], l [S,H,1], m [S,H,1])."""
    H, _, D = q_b.shape
    G, Tk, _ = k.shape
    rep = H // G
    kk = torch.repeat_interleave(k.to(torch.float32), rep, 0)
    vv = torch.repeat_interleave(v.to(torch.float32), rep, 0)
    s = (q_b.to(torch.float32) * scale) @ kk.transpose(-1, -2) * math.log2(math.e)   # [H,1,Tk]
    nblk = (Tk + block - 1) // block
    bps = (nblk + num_splits - 1) // num_splits
    acc = torch.zeros(num_splits, H, 1, D)
    l = torch.zeros(num_splits, H, 1)
    m = torch.full((num_splits, H, 1), float("-inf"))
    for i in range(num_splits):
        lo, hi = min(Tk, i * bps * block), min(Tk, (i + 1) * bps * block)
        if hi <= lo:
            continue
        si = s[:, :, lo:hi]
        mi = si.amax(-1)
        p = torch.exp2(si - mi[..., None])
        m[i], l[i], acc[i] = mi, p.sum(-1), p @ vv[:, lo:hi]
    return acc, l, m


def select_kv_splits(ctx_window_size: int, max_kv_splits: int, phase: int, tq: int) -> int:
    """The reference's static split policy (fa2.py:201-212)."""
    if phase != PHASE_DECODE or tq != 1:
        return 1
    if max_kv_splits <= 1 or ctx_window_size <= 4096:
        target = 1
    elif ctx_window_size < 8192:
        target = 4
    elif ctx_window_size < 32768:
        target = 8
    else:
        target = 16
    return max(1, min(target, max_kv_splits))


def add_kv_to_cache_fp8(x, cache_u8, scales, cache_offsets, rmsnorm_eps, x_rsos=None, user_phase=None, phase=0, *,
                        block_tables, page_size=16, headroom=2.0):
    """Returns (pool bytes, scales) after the append (copies).  Row p = off[b] + t of slot b goes
    to page block_tables[b, p // page], row p % page; the page's scale is
    max(max|first row| * headroom / 448, 2^-24), taken from the page's first row whichever call
    appends it, and a row is stored as the round-to-nearest-even, saturating e4m3 of row / scale
    (fp32 arithmetic throughout)."""
    pool = cache_u8.detach().clone().view(torch.uint8)
    sc = scales.detach().clone()
    B, G, Tq, D = x.shape
    xf = x.detach().to(torch.float32)
    if x_rsos is not None:
        xf = xf * (1.0 / torch.sqrt(x_rsos.detach().to(torch.float32) / D + rmsnorm_eps))[..., None]
    for b in range(B):
        if user_phase is not None and int(user_phase[b]) != int(phase):
            continue
        off = int(cache_offsets[b])
        for t in range(Tq):
            pos = off + t
            page, row = int(block_tables[b, pos // page_size]), pos % page_size
            t0 = t - row
            for g in range(G):
                if t0 >= 0:
                    amax = xf[b, g, t0].abs().max()
                    s = torch.maximum(amax * torch.tensor(headroom, dtype=torch.float32) / 448.0,
                                      torch.tensor(2.0 ** -24, dtype=torch.float32))
                    if row == 0:
                        sc[page, g] = s
                else:
                    s = sc[page, g]
                q = torch.clamp(xf[b, g, t] / s, -448.0, 448.0).to(torch.float8_e4m3fn)
                pool[page, g, row] = q.view(torch.uint8)
    return pool, sc


def dequantise_fp8_pool(pool_u8, scales) -> torch.Tensor:
    """[num_pages,G,page,D] bytes + [num_pages,G] scales -> fp32 values e4m3(byte) * scale."""
    return pool_u8.view(torch.float8_e4m3fn).to(torch.float32) * scales.to(torch.float32)[:, :, None, None]
