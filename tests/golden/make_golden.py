"""Generates tests/golden/*.npz from the reference's own torch implementation.

Run in the build container only (needs the reference checkout):
    python tests/golden/make_golden.py
Every case drives scripts/reference_impl.py's LayerKVCache (add / retrieve, :421-475) exactly
as Attention.forward does (:210-237: add the new K/V, then retrieve with the new queries),
on seeded inputs that are first rounded to fp16 so they are stored exactly in 2 bytes.
Stored per case: the inputs (fp16), the reference output (fp32) and the case parameters.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import ref_loader  # noqa: E402

OUT = Path(__file__).resolve().parent


def rnd(gen, *shape):
    return torch.randn(*shape, generator=gen).to(torch.float16).to(torch.float32)


def run_case(name, *, heads, kv_heads, head_dim, context_length, sliding_window, is_swa, chunks,
             scale, seed):
    """chunks: list of (phase, n_tokens); the output of the LAST chunk is stored, together
    with all K/V fed in (the cache content) and the last chunk's queries."""
    gen = torch.Generator().manual_seed(seed)
    cache = ref_loader.make_layer_cache(heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                        context_length=context_length, sliding_window=sliding_window,
                                        is_swa=is_swa)
    ks, vs = [], []
    out = q = None
    for phase, n in chunks:
        if phase == "prefill":
            cache.set_prefill()
        else:
            cache.set_decode()
        k = rnd(gen, 1, kv_heads, n, head_dim)
        v = rnd(gen, 1, kv_heads, n, head_dim)
        q = rnd(gen, 1, heads, n, head_dim)
        cache.add(k, v)
        out = cache.retrieve(q * scale)
        ks.append(k)
        vs.append(v)
    np.savez(
        OUT / f"{name}.npz",
        q=q[0].numpy().astype(np.float16),
        k_all=torch.cat(ks, 2)[0].numpy().astype(np.float16),
        v_all=torch.cat(vs, 2)[0].numpy().astype(np.float16),
        out=out[0].numpy().astype(np.float32),
        scale=np.float32(scale),
        window=np.int32(sliding_window if is_swa else context_length),
        is_swa=np.int32(is_swa),
        last_chunk=np.int32(chunks[-1][1]),
        last_phase=np.int32(1 if chunks[-1][0] == "prefill" else 2),
    )
    print(name, tuple(out.shape), float(out.abs().mean()))


def run_rope_case(name, *, heads, kv_heads, head_dim, n_tokens, base_time_offset, is_swa, freq_base, seed):
    """q/k/v of one chunk through the reference's q_norm/k_norm/v_norm and RoPE, in the order
    of Attention.forward (reference_impl.py:219-233).  A global layer divides its frequencies by
    the model's rope_freqs factors (reference_impl.py:246-247)."""
    gen = torch.Generator().manual_seed(seed)
    eps = 1e-6
    q_w = (1.0 + 0.25 * rnd(gen, head_dim)).to(torch.float16).to(torch.float32)
    k_w = (1.0 + 0.25 * rnd(gen, head_dim)).to(torch.float16).to(torch.float32)
    factors = None if is_swa else (1.0 + torch.rand(head_dim // 2, generator=gen) * 7.0)
    rope, q_norm, k_norm, v_norm = ref_loader.make_rope_and_norms(
        head_dim=head_dim, is_swa=is_swa, freq_base=freq_base, eps=eps, rope_freqs=factors,
        q_weight=q_w, k_weight=k_w)
    q = 4.0 * rnd(gen, 1, heads, n_tokens, head_dim)
    k = 0.5 * rnd(gen, 1, kv_heads, n_tokens, head_dim)
    v = 2.0 * rnd(gen, 1, kv_heads, n_tokens, head_dim)
    (q_out,) = rope(q_norm(q), base_time_offset=base_time_offset)
    (k_out,) = rope(k_norm(k), base_time_offset=base_time_offset)
    v_out = v_norm(v)
    np.savez(
        OUT / f"{name}.npz",
        q=q[0].numpy().astype(np.float16), k=k[0].numpy().astype(np.float16), v=v[0].numpy().astype(np.float16),
        q_w=q_w.numpy().astype(np.float16), k_w=k_w.numpy().astype(np.float16),
        freqs=rope.freqs.numpy().astype(np.float32),
        q_out=q_out[0].numpy().astype(np.float32), k_out=k_out[0].numpy().astype(np.float32),
        v_out=v_out[0].numpy().astype(np.float32),
        base_time_offset=np.int32(base_time_offset), eps=np.float32(eps),
    )
    print(name, tuple(q_out.shape), float(q_out.abs().mean()))


def main():
    # norm + rotary embedding ahead of the append: a sliding-window layer (plain frequencies)
    # and a global layer (frequencies divided by per-pair factors), at small and large positions
    run_rope_case("rope_swa", heads=4, kv_heads=2, head_dim=256, n_tokens=9, base_time_offset=0,
                  is_swa=True, freq_base=10000.0, seed=21)
    run_rope_case("rope_global_far", heads=4, kv_heads=2, head_dim=256, n_tokens=5, base_time_offset=100000,
                  is_swa=False, freq_base=1000000.0, seed=22)
    run_rope_case("rope_d128", heads=2, kv_heads=1, head_dim=128, n_tokens=4, base_time_offset=37,
                  is_swa=True, freq_base=10000.0, seed=23)
    common = dict(heads=4, kv_heads=2, head_dim=256)
    # fresh causal prefill, global layer, BASELINE scale 1/sqrt(256)
    run_case("prefill_causal", **common, context_length=64, sliding_window=16, is_swa=False,
             chunks=[("prefill", 40)], scale=1 / 16, seed=11)
    # the reference's own setting: no softmax scale (fa2.py:89, reference_impl.py:443)
    run_case("prefill_causal_unscaled", **common, context_length=64, sliding_window=16, is_swa=False,
             chunks=[("prefill", 24)], scale=1.0, seed=12)
    # sliding-window prefill longer than the window: per-query mask (reference_impl.py:440-441)
    run_case("prefill_swa", **common, context_length=64, sliding_window=16, is_swa=True,
             chunks=[("prefill", 40)], scale=1 / 16, seed=13)
    # chunked prefill: second chunk attends to the first through the cache
    run_case("prefill_chunked", **common, context_length=64, sliding_window=16, is_swa=False,
             chunks=[("prefill", 24), ("prefill", 16)], scale=1 / 16, seed=14)
    # decode after prefill, global layer
    run_case("decode_global", **common, context_length=64, sliding_window=16, is_swa=False,
             chunks=[("prefill", 39), ("decode", 1)], scale=1 / 16, seed=15)
    # decode on a sliding-window layer whose context is longer than the window
    run_case("decode_swa", **common, context_length=64, sliding_window=16, is_swa=True,
             chunks=[("prefill", 39), ("decode", 1)], scale=1 / 16, seed=16)
    # the CPU-reference configuration of the benchmark (B1 S512 H8 G2 D256), sub-sampled rows
    gen = torch.Generator().manual_seed(0)
    cache = ref_loader.make_layer_cache(heads=8, kv_heads=2, head_dim=256, context_length=512,
                                        sliding_window=512, is_swa=False)
    q = rnd(gen, 1, 8, 512, 256)
    k = rnd(gen, 1, 2, 512, 256)
    v = rnd(gen, 1, 2, 512, 256)
    cache.set_prefill()
    cache.add(k, v)
    out = cache.retrieve(q * (1 / 16))
    rows = np.arange(0, 512, 37)
    np.savez(OUT / "config1_rows.npz", rows=rows.astype(np.int32), out_rows=out[0][:, rows].numpy(),
             seed=np.int32(0), in_checksum=np.float64(float(q.double().sum() + k.double().sum() + v.double().sum())))
    print("config1_rows", out.shape)


if __name__ == "__main__":
    main()
