"""Imports the reference's torch implementation (scripts/reference_impl.py) unmodified.

TEST INFRASTRUCTURE ONLY.  Works only where the reference checkout is mounted (the build
container); it is used to pin the oracle and to generate tests/golden/*.npz, never at run
time on a GPU box and never by the product.

Why a shim: the file does ``from g4b import gguf`` (reference_impl.py:19), and the package
``__init__`` pulls ``cuda.core`` which is not installed; and it refers to the ``KVCaches``
alias in an annotation before defining it (reference_impl.py:210 vs :482), which needs lazily
evaluated annotations.  So: register an empty ``g4b`` package whose ``__path__`` points at
the reference, load ``g4b/gguf.py`` by path, and exec the script with the
``from __future__ import annotations`` compiler flag.
"""
from __future__ import annotations

import __future__ as _future
import importlib.util
import os
import sys
import types
from pathlib import Path

def _find_reference_root() -> Path:
    """$G4B_REFERENCE_ROOT, else the byte copies that oracle/make_ref.py leaves under
    oracle/_ref/ (they travel to a GPU box), else a checkout named ``reference`` beside the
    repository."""
    here = Path(__file__).resolve().parent
    cands = [os.environ.get("G4B_REFERENCE_ROOT"), str(here / "_ref"), str(here.parents[1] / "reference")]
    for c in cands:
        if c and (Path(c) / "scripts" / "reference_impl.py").exists():
            return Path(c)
    return here / "_ref"


REFERENCE_ROOT = _find_reference_root()


def available() -> bool:
    return (REFERENCE_ROOT / "scripts" / "reference_impl.py").exists()


def load_reference_impl():
    """Returns the reference_impl module (LayerKVCache, Gemma4Config, ...)."""
    name = "_g4b_reference_impl"
    if name in sys.modules:
        return sys.modules[name]
    if not available():
        raise RuntimeError(f"reference checkout not found under {REFERENCE_ROOT}")
    if "g4b" not in sys.modules:
        pkg = types.ModuleType("g4b")
        pkg.__path__ = [str(REFERENCE_ROOT / "g4b")]
        sys.modules["g4b"] = pkg
    if "g4b.gguf" not in sys.modules:
        spec = importlib.util.spec_from_file_location("g4b.gguf", REFERENCE_ROOT / "g4b" / "gguf.py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules["g4b.gguf"] = mod
        spec.loader.exec_module(mod)
        sys.modules["g4b"].gguf = mod
    path = REFERENCE_ROOT / "scripts" / "reference_impl.py"
    module = types.ModuleType(name)
    module.__file__ = str(path)
    sys.modules[name] = module
    code = compile(path.read_text(), str(path), "exec",
                   flags=_future.annotations.compiler_flag, dont_inherit=True)
    exec(code, module.__dict__)
    return module


def make_layer_cache(*, heads: int, kv_heads: int, head_dim: int, context_length: int,
                     sliding_window: int, is_swa: bool):
    """A reference LayerKVCache (reference_impl.py:396-479) for one attention layer."""
    ref = load_reference_impl()
    conf = ref.Gemma4Config(
        block_count=1, context_length=context_length, embedding_length=heads * head_dim,
        feed_forward_length=1, attention_head_count=heads, attention_head_count_kv=kv_heads,
        rope_freq_base=10000.0, rope_freq_base_swa=10000.0, attention_layer_norm_rms_epsilon=1e-6,
        attention_key_length=head_dim, attention_value_length=head_dim, final_logit_softcapping=0.0,
        attention_sliding_window=sliding_window, attention_shared_kv_layers=0,
        embedding_length_per_layer_input=0, attention_sliding_window_pattern=[is_swa],
        attention_key_length_swa=head_dim, attention_value_length_swa=head_dim,
        rope_dimension_count=head_dim, rope_dimension_count_swa=head_dim,
    )
    return ref.LayerKVCache(conf, 0)


def make_rope_and_norms(*, head_dim: int, is_swa: bool, freq_base: float, eps: float, rope_freqs=None,
                        q_weight=None, k_weight=None):
    """The reference's RoPE (reference_impl.py:240-265) and its q / k / v RMSNorm modules
    (reference_impl.py:77-85; the V norm has no weight) as Attention.forward uses them
    (reference_impl.py:219-233)."""
    ref = load_reference_impl()
    conf = ref.Gemma4Config(
        block_count=1, context_length=1, embedding_length=head_dim,
        feed_forward_length=1, attention_head_count=1, attention_head_count_kv=1,
        rope_freq_base=freq_base, rope_freq_base_swa=freq_base, attention_layer_norm_rms_epsilon=eps,
        attention_key_length=head_dim, attention_value_length=head_dim, final_logit_softcapping=0.0,
        attention_sliding_window=1, attention_shared_kv_layers=0,
        embedding_length_per_layer_input=0, attention_sliding_window_pattern=[is_swa],
        attention_key_length_swa=head_dim, attention_value_length_swa=head_dim,
        rope_dimension_count=head_dim, rope_dimension_count_swa=head_dim,
    )
    rope = ref.RoPE(conf, None if is_swa else rope_freqs)
    return rope, ref.RMSNorm(conf, q_weight), ref.RMSNorm(conf, k_weight), ref.RMSNorm(conf, None)
