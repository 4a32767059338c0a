"""Reference-generated decode fixtures reproduced on the GPU: append through the C ABI into
ring and paged caches, then decode attention."""
from pathlib import Path

import numpy as np
import pytest
import torch

from g4b_b200.kernels import fa2
from g4b_b200.kernels.add_kv_to_cache import add_kv_to_cache
from helpers import assert_close

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["decode_global", "decode_swa"])
@pytest.mark.parametrize("layout", ["ring", "ring_wrapped", "paged"])
def test_decode_matches_reference_golden(cuda, name, layout):
    z = np.load(GOLD / f"{name}.npz")
    q = torch.from_numpy(z["q"])[None].to(cuda)            # [1,H,1,D] fp16
    k_all = torch.from_numpy(z["k_all"])[None].to(cuda)    # [1,G,n,D]
    v_all = torch.from_numpy(z["v_all"])[None].to(cuda)
    _, G, n_all, D = k_all.shape
    is_swa, window = bool(z["is_swa"]), int(z["window"])
    o = torch.zeros_like(q)
    time = torch.tensor([n_all], dtype=torch.int32, device=cuda)
    off = torch.zeros(1, dtype=torch.int32, device=cuda)
    if layout == "paged":
        n_pages = (n_all + 15) // 16
        perm = torch.randperm(n_pages + 2, generator=torch.Generator().manual_seed(1))[:n_pages]
        bt = perm.to(torch.int32)[None].to(cuda)
        kp = torch.full((n_pages + 2, G, 16, D), float("nan"), dtype=torch.float16, device=cuda)
        vp = torch.full_like(kp, float("nan"))
        add_kv_to_cache(k_all, kp, off, 1e-6, block_tables=bt)
        add_kv_to_cache(v_all, vp, off, 1e-6, block_tables=bt)
        fa2.flash_attention(q, kp, vp, o, time, None, n_pages * 16, 2, scale=float(z["scale"]),
                            sliding_window=window if is_swa else None, block_tables=bt)
    else:
        if layout == "ring_wrapped":
            if not is_swa:
                pytest.skip("a global layer's ring does not wrap while the context fits")
            T = window            # decode: Tq = 1, the ring holds exactly the window
        else:
            T = 64
        kc = torch.zeros(1, G, T, D, dtype=torch.float16, device=cuda)
        vc = torch.zeros_like(kc)
        # feed the context in ring-sized pieces, as chunked prefill would
        at = 0
        while at < n_all:
            n = min(T, n_all - at)
            add_kv_to_cache(k_all[:, :, at:at + n], kc, off + at, 1e-6)
            add_kv_to_cache(v_all[:, :, at:at + n], vc, off + at, 1e-6)
            at += n
        ctx_window = window if is_swa else T
        fa2.flash_attention(q, kc, vc, o, time, None, ctx_window, 2, scale=float(z["scale"]))
    assert_close(o[0].cpu(), torch.from_numpy(z["out"]), f"{name}/{layout}")
