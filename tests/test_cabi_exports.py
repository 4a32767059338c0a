"""The C-ABI library loads without a GPU, exports every symbol include/g4b_attn.h declares,
and rejects bad arguments before touching CUDA."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from g4b_b200 import _cabi
from g4b_b200.kernels import add_kv_to_cache as akv
from g4b_b200.kernels import advance_decode_state as ads
from g4b_b200.kernels import fa2
from helpers import orc

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "g4b_attn.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(g4b_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = ctypes.CDLL(str(_cabi.lib_path()))
    names = declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in g4b_attn.h but not exported"
    assert set(names) == set(_cabi.EXPORTS), "ctypes table and header disagree"


def test_abi_version_and_split_policy():
    lib = _cabi.load()
    assert lib.g4b_abi_version() == 2
    for w in (1, 1024, 4096, 4097, 8191, 8192, 32767, 32768, 131072):
        for cap in (1, 2, 4, 8, 16, 64):
            for phase, tq in ((2, 1), (1, 1), (2, 2)):
                assert fa2.select_kv_splits(w, cap, phase, tq) == orc.select_kv_splits(w, cap, phase, tq)


def test_constants_match_reference():
    # g4b/kernels/fa2.py:14-16,29-31
    assert (fa2.STAGE_FULL, fa2.STAGE_ON_BAND, fa2.STAGE_CAUSAL) == (1, 2, 3)
    assert (fa2.PHASE_UNALLOCATED, fa2.PHASE_PREFILL, fa2.PHASE_DECODE) == (0, 1, 2)


def _attn_inputs(B=2, H=8, G=2, Tq=1, T=64, D=256, dtype=torch.float16):
    q = torch.zeros(B, H, Tq, D, dtype=dtype)
    k = torch.zeros(B, G, T, D, dtype=dtype)
    v = torch.zeros(B, G, T, D, dtype=dtype)
    o = torch.zeros(B, H, Tq, D, dtype=dtype)
    time = torch.full((B,), T, dtype=torch.int32)
    phase = torch.full((B,), 2, dtype=torch.uint8)
    return q, k, v, o, time, phase


def test_partial_triple_must_be_complete():
    # fa2.py:656-657
    q, k, v, o, time, phase = _attn_inputs()
    po = torch.zeros(4, 2, 8, 1, 256)
    with pytest.raises(ValueError, match="provided together"):
        fa2.flash_attention(q, k, v, o, time, phase, 64, 2, po, None, None, stream=0)


@pytest.mark.parametrize("breaker,match", [
    (lambda a: a.__setitem__("q", a["q"][..., :128]), "o shape|head dim"),
    (lambda a: a.__setitem__("k", a["k"][:, :, :, ::2]), "innermost stride"),
    (lambda a: a.__setitem__("time", a["time"].to(torch.int64)), "int32"),
    (lambda a: a.__setitem__("ctx", 65), "exceeds cache length"),        # fa2.py:298
    (lambda a: a.__setitem__("phase_t", a["phase_t"].to(torch.int32)), "uint8"),
    (lambda a: a.__setitem__("k", a["k"].to(torch.float32)), "f16|bf16"),
    (lambda a: a.__setitem__("stage", 2), "stage"),
])
def test_attention_rejects_bad_arguments(breaker, match):
    q, k, v, o, time, phase = _attn_inputs()
    a = dict(q=q, k=k, v=v, o=o, time=time, phase_t=phase, ctx=64, stage=3)
    breaker(a)
    with pytest.raises(ValueError, match=match):
        fa2.flash_attention(a["q"], a["k"], a["v"], a["o"], a["time"], a["phase_t"], a["ctx"], 2,
                            stage=a["stage"], stream=0)


def test_head_dims_outside_the_built_ones_are_unsupported():
    """Tq == 1 takes head dims 128, 256 and 512; Tq > 1 takes 128 and 256."""
    for D, Tq, ok in ((128, 1, True), (512, 1, True), (64, 1, False), (128, 2, True), (64, 2, False), (512, 2, False), (256, 2, True)):
        q, k, v, o, time, phase = _attn_inputs(D=D, Tq=Tq)
        call = lambda: fa2.flash_attention(q, k, v, o, time, phase, 64, 2 if Tq == 1 else 1, stream=0)
        if ok:
            call()
        else:
            with pytest.raises(ValueError, match="head dim"):
                call()


def test_append_rejects_bad_arguments():
    x = torch.zeros(2, 2, 3, 256)
    cache = torch.zeros(2, 2, 17, 256, dtype=torch.float16)
    off = torch.zeros(2, dtype=torch.int32)
    with pytest.raises(ValueError, match="cache_offsets"):
        akv.add_kv_to_cache(x, cache, off[:1], 1e-6, stream=0)
    with pytest.raises(ValueError, match="more new tokens"):   # add_kv_to_cache.py:123
        akv.add_kv_to_cache(torch.zeros(2, 2, 18, 256), cache, off, 1e-6, stream=0)
    with pytest.raises(ValueError, match="kv heads or head dim"):
        akv.add_kv_to_cache(torch.zeros(2, 4, 3, 256), cache, off, 1e-6, stream=0)
    with pytest.raises(ValueError, match="x_rsos"):
        akv.add_kv_to_cache(x, cache, off, 1e-6, torch.zeros(2, 2, 4), stream=0)
    with pytest.raises(TypeError):
        akv.add_kv_to_cache(object(), cache, off, 1e-6, stream=0)


def test_advance_rejects_bad_arguments():
    i32 = lambda *s: torch.zeros(*s, dtype=torch.int32)
    with pytest.raises(ValueError, match="B entries"):
        ads.advance_decode_state(i32(1, 4), i32(4, 1), i32(3), i32(4), torch.zeros(4, dtype=torch.uint8), stream=0)
    with pytest.raises(ValueError, match="int32"):
        ads.advance_decode_state(i32(1, 4), i32(4, 1), i32(4), i32(4), i32(4), stream=0)


def test_tensor_like_duck_typing():
    """Anything with shape/stride/dtype/data_ptr is accepted, stride as a tuple or a callable
    (g4b/kernels/utils.py:51-60)."""
    class Fake:
        def __init__(self, t, as_tuple):
            self.shape, self.dtype, self._t = tuple(t.shape), "float16", t
            self.stride = tuple(t.stride()) if as_tuple else t.stride
        def data_ptr(self):
            return self._t.data_ptr()
    t = torch.zeros(2, 3, 4, dtype=torch.float16).permute(1, 0, 2)
    for as_tuple in (True, False):
        c = _cabi.as_tensor(Fake(t, as_tuple))
        assert list(c.shape[:3]) == [3, 2, 4] and list(c.stride[:3]) == [4, 12, 1]
        assert c.dtype == _cabi.F16 and c.ndim == 3
    assert _cabi.as_tensor(None).ptr is None


def test_exchange_buffer_sizes_host_only():
    """g4b_exchange_buffer_bytes is pure host arithmetic: 2 parities x world x rows x slices x
    (columns + l + m) words of 8 bytes (value, launch count), the larger of the two entry points'
    layouts (32-column slices for g4b_attn_combine_exchange, 8-column slices for
    g4b_decode_step)."""
    lib = _cabi.load()
    assert lib.g4b_exchange_buffer_bytes(8, 8, 256) == 2 * 8 * 8 * 32 * 10 * 8
    assert lib.g4b_exchange_buffer_bytes(2, 3, 40) == 2 * 2 * 3 * 2 * 34 * 8      # 2 slices of 32 > 5 slices of 8


def test_valid_arguments_pass_validation_without_a_launch():
    """In validate-only mode a call whose arguments pass every check returns normally and
    launches nothing (there is no GPU here to launch on)."""
    q, k, v, o, time, phase = _attn_inputs()
    fa2.flash_attention(q, k, v, o, time, phase, 64, 2, stream=0)
    po, pl = torch.zeros(4, 2, 8, 1, 256), torch.zeros(4, 2, 8, 1)
    fa2.flash_attention(q, k, v, o, time, phase, 64, 2, po, pl, pl.clone(), num_kv_splits=4, stream=0)
    akv.add_kv_to_cache(torch.zeros(2, 2, 3, 256), torch.zeros(2, 2, 17, 256, dtype=torch.float16),
                        torch.zeros(2, dtype=torch.int32), 1e-6, stream=0)
    assert o.abs().sum() == 0


@pytest.mark.launches_allowed
def test_host_and_foreign_device_tensors_are_refused():
    """Outside validate-only mode the wrappers refuse torch tensors that are not on the
    current CUDA device before anything reaches the library."""
    q, k, v, o, time, phase = _attn_inputs()
    with pytest.raises(ValueError, match="CUDA tensor"):
        fa2.flash_attention(q, k, v, o, time, phase, 64, 2, stream=0)
    with pytest.raises(ValueError, match="CUDA tensor"):
        akv.add_kv_to_cache(torch.zeros(2, 2, 3, 256), torch.zeros(2, 2, 17, 256, dtype=torch.float16),
                            torch.zeros(2, dtype=torch.int32), 1e-6, stream=0)


def test_fp8_dequant_rejects_bad_arguments():
    pool = torch.zeros(6, 2, 16, 256, dtype=torch.uint8)
    sc = torch.zeros(6, 2)
    out = torch.zeros(6, 2, 16, 256, dtype=torch.float16)
    akv.dequantise_fp8_pool(pool, sc, out, stream=0)                    # valid: passes, launches nothing
    bt, time = torch.zeros(2, 3, dtype=torch.int32), torch.zeros(2, dtype=torch.int32)
    akv.dequantise_fp8_pool(pool, sc, out, block_tables=bt, time_dim_sizes=time, user_phase=torch.zeros(2, dtype=torch.uint8),
                            phase=1, stream=0)
    with pytest.raises(ValueError, match="shape of cache"):
        akv.dequantise_fp8_pool(pool, sc, out[:5], stream=0)
    with pytest.raises(ValueError, match="f16 or bf16"):
        akv.dequantise_fp8_pool(pool, sc, out.float(), stream=0)
    with pytest.raises(ValueError, match="one byte"):
        akv.dequantise_fp8_pool(out, sc, out, stream=0)
    with pytest.raises(ValueError, match=r"\[num_pages, G\]"):
        akv.dequantise_fp8_pool(pool, sc[:, :1], out, stream=0)
    with pytest.raises(ValueError, match="needs time_dim_sizes"):
        akv.dequantise_fp8_pool(pool, sc, out, block_tables=bt, stream=0)
    with pytest.raises(ValueError, match="only read with block_tables"):
        akv.dequantise_fp8_pool(pool, sc, out, time_dim_sizes=time, stream=0)
    with pytest.raises(ValueError, match="page_size"):
        akv.dequantise_fp8_pool(pool, sc, out, page_size=32, stream=0)
