"""ctypes binding of libg4b_attn.so (declared in include/g4b_attn.h).

The library is the product: if it is missing or cannot be loaded every op raises, there is
no fallback path.  Tensor-like arguments are anything with ``.shape``, ``.stride`` (a
sequence or a callable), ``.dtype`` and ``.data_ptr()``, which is what the reference's
launcher accepts (g4b/kernels/utils.py:51-60,113-122).
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libg4b_attn.so"

# enum G4bDtype
F32, F16, BF16, I32, I64, U8, FP8_E4M3 = 0, 1, 2, 3, 4, 5, 6

_DTYPE_NAMES = {
    "float32": F32, "f32": F32, "float": F32,
    "float16": F16, "f16": F16, "half": F16,
    "bfloat16": BF16, "bf16": BF16,
    "int32": I32, "i32": I32,
    "int64": I64, "i64": I64, "long": I64,
    "uint8": U8, "u8": U8,
    "float8_e4m3fn": FP8_E4M3, "fp8_e4m3": FP8_E4M3,
}


class G4bTensor(ctypes.Structure):
    _fields_ = [
        ("ptr", ctypes.c_void_p),
        ("shape", ctypes.c_int64 * 5),
        ("stride", ctypes.c_int64 * 5),
        ("ndim", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
    ]


class G4bAttnArgs(ctypes.Structure):
    _fields_ = [
        ("q", G4bTensor), ("k_cache", G4bTensor), ("v_cache", G4bTensor), ("o", G4bTensor),
        ("time_dim_sizes", G4bTensor), ("user_phase", G4bTensor),
        ("partial_o", G4bTensor), ("partial_l", G4bTensor), ("partial_m", G4bTensor),
        ("block_tables", G4bTensor),
        ("ctx_window_size", ctypes.c_int32), ("phase", ctypes.c_int32), ("stage", ctypes.c_int32),
        ("page_size", ctypes.c_int32), ("sliding_window", ctypes.c_int32),
        ("num_kv_splits", ctypes.c_int32), ("scale", ctypes.c_float), ("reserved", ctypes.c_int32),
    ]


class G4bCombineArgs(ctypes.Structure):
    _fields_ = [
        ("partial_o", G4bTensor), ("partial_l", G4bTensor), ("partial_m", G4bTensor), ("o", G4bTensor),
        ("user_phase", G4bTensor), ("num_splits", ctypes.c_int32), ("phase", ctypes.c_int32),
    ]


class G4bAppendArgs(ctypes.Structure):
    _fields_ = [
        ("x", G4bTensor), ("cache", G4bTensor), ("cache_offsets", G4bTensor), ("x_rsos", G4bTensor),
        ("user_phase", G4bTensor), ("block_tables", G4bTensor),
        ("rmsnorm_eps", ctypes.c_float), ("phase", ctypes.c_int32), ("page_size", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
    ]


class G4bRopeAppendArgs(ctypes.Structure):
    _fields_ = [
        ("q", G4bTensor), ("k", G4bTensor), ("v", G4bTensor), ("q_out", G4bTensor), ("k_out", G4bTensor),
        ("rope_freqs", G4bTensor), ("cache_offsets", G4bTensor),
        ("q_rsos", G4bTensor), ("k_rsos", G4bTensor), ("v_rsos", G4bTensor),
        ("q_norm_w", G4bTensor), ("k_norm_w", G4bTensor),
        ("k_cache", G4bTensor), ("v_cache", G4bTensor),
        ("user_phase", G4bTensor), ("block_tables", G4bTensor),
        ("rmsnorm_eps", ctypes.c_float), ("phase", ctypes.c_int32), ("page_size", ctypes.c_int32),
        ("norm_qk", ctypes.c_int32), ("norm_v", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


class G4bExchangeArgs(ctypes.Structure):
    _fields_ = [
        ("partial_o", G4bTensor), ("partial_l", G4bTensor), ("partial_m", G4bTensor), ("o", G4bTensor),
        ("user_phase", G4bTensor),
        ("xbuf", ctypes.c_void_p * 8), ("state", ctypes.c_void_p),
        ("xbuf_bytes", ctypes.c_int64),
        ("num_splits", ctypes.c_int32), ("phase", ctypes.c_int32), ("world", ctypes.c_int32), ("rank", ctypes.c_int32),
    ]


class G4bDecodeStepArgs(ctypes.Structure):
    _fields_ = [
        ("attn", G4bAttnArgs), ("k_new", G4bTensor), ("v_new", G4bTensor),
        ("xbuf", ctypes.c_void_p * 8), ("state", ctypes.c_void_p), ("xbuf_bytes", ctypes.c_int64),
        ("world", ctypes.c_int32), ("rank", ctypes.c_int32),
    ]


class G4bFp8AppendArgs(ctypes.Structure):
    _fields_ = [
        ("x", G4bTensor), ("cache", G4bTensor), ("scales", G4bTensor), ("cache_offsets", G4bTensor),
        ("x_rsos", G4bTensor), ("user_phase", G4bTensor), ("block_tables", G4bTensor),
        ("rmsnorm_eps", ctypes.c_float), ("headroom", ctypes.c_float), ("phase", ctypes.c_int32),
        ("page_size", ctypes.c_int32),
    ]


class G4bFp8DequantArgs(ctypes.Structure):
    _fields_ = [
        ("cache", G4bTensor), ("scales", G4bTensor), ("out", G4bTensor), ("block_tables", G4bTensor),
        ("time_dim_sizes", G4bTensor), ("user_phase", G4bTensor), ("phase", ctypes.c_int32), ("page_size", ctypes.c_int32),
    ]


class G4bAdvanceArgs(ctypes.Structure):
    _fields_ = [
        ("input_token_ids", G4bTensor), ("out_token_ids", G4bTensor), ("cache_offsets", G4bTensor),
        ("time_dim_sizes", G4bTensor), ("user_phase", G4bTensor),
    ]


# every symbol include/g4b_attn.h declares: name -> (restype, argtypes)
EXPORTS = {
    "g4b_flash_attention": (ctypes.c_int, [ctypes.POINTER(G4bAttnArgs), ctypes.c_void_p]),
    "g4b_attn_prefill": (ctypes.c_int, [ctypes.POINTER(G4bAttnArgs), ctypes.c_void_p]),
    "g4b_attn_decode": (ctypes.c_int, [ctypes.POINTER(G4bAttnArgs), ctypes.c_void_p]),
    "g4b_attn_decode_static_scratch": (ctypes.c_int, [ctypes.POINTER(G4bAttnArgs), ctypes.c_void_p]),
    "g4b_decode_step": (ctypes.c_int, [ctypes.POINTER(G4bDecodeStepArgs), ctypes.c_void_p]),
    "g4b_kv_append_fp8": (ctypes.c_int, [ctypes.POINTER(G4bFp8AppendArgs), ctypes.c_void_p]),
    "g4b_kv_dequant_fp8": (ctypes.c_int, [ctypes.POINTER(G4bFp8DequantArgs), ctypes.c_void_p]),
    "g4b_flash_attention_fp8": (ctypes.c_int, [ctypes.POINTER(G4bAttnArgs), ctypes.POINTER(G4bTensor),
                                               ctypes.POINTER(G4bTensor), ctypes.c_void_p]),
    "g4b_attn_combine": (ctypes.c_int, [ctypes.POINTER(G4bCombineArgs), ctypes.c_void_p]),
    "g4b_attn_combine_exchange": (ctypes.c_int, [ctypes.POINTER(G4bExchangeArgs), ctypes.c_void_p]),
    "g4b_exchange_buffer_bytes": (ctypes.c_int64, [ctypes.c_int, ctypes.c_int64, ctypes.c_int]),
    "g4b_select_kv_splits": (ctypes.c_int, [ctypes.c_int] * 4),
    "g4b_kv_append": (ctypes.c_int, [ctypes.POINTER(G4bAppendArgs), ctypes.c_void_p]),
    "g4b_rope_norm_append": (ctypes.c_int, [ctypes.POINTER(G4bRopeAppendArgs), ctypes.c_void_p]),
    "g4b_advance_decode_state": (ctypes.c_int, [ctypes.POINTER(G4bAdvanceArgs), ctypes.c_void_p]),
    "g4b_last_error_string": (ctypes.c_char_p, []),
    "g4b_abi_version": (ctypes.c_int, []),
    "g4b_device_status": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]),
    "g4b_set_validate_only": (None, [ctypes.c_int]),
}

_lib = None


def lib_path() -> Path:
    return Path(os.environ.get("G4B_B200_LIB", str(_LIB_PATH)))


def load() -> ctypes.CDLL:
    """Loads the library once; raises if it has not been built (python -m g4b_b200.build)."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: build it with `python -m g4b_b200.build` (needs nvcc). "
                "There is no fallback implementation."
            )
        lib = ctypes.CDLL(str(path))
        for name, (restype, argtypes) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def dtype_code(dt) -> int:
    name = getattr(dt, "name", None) or str(dt)
    name = name.replace("torch.", "").replace("numpy.", "").lower()
    if name not in _DTYPE_NAMES:
        raise TypeError(f"unsupported dtype {dt!r}")
    return _DTYPE_NAMES[name]


def _strides(t) -> list[int]:
    if isinstance(t.stride, (list, tuple)):
        return list(t.stride)
    if callable(t.stride):
        return [t.stride(i) for i in range(len(t.shape))]
    raise RuntimeError("Failed to normalize tensor stride into list[int]")


_validate_only_depth = 0


class validate_only:
    """``with _cabi.validate_only():`` -- the library checks arguments and launches nothing
    (g4b_set_validate_only), and the wrappers accept host tensors.  For tests of the argument
    checks on machines without a GPU; a call that passes every check returns normally."""

    def __enter__(self):
        global _validate_only_depth
        _validate_only_depth += 1
        load().g4b_set_validate_only(1)
        return self

    def __exit__(self, *exc):
        global _validate_only_depth
        _validate_only_depth -= 1
        if _validate_only_depth == 0:
            load().g4b_set_validate_only(0)
        return False


def _check_device(t) -> None:
    """A kernel given a host pointer, or a pointer into another GPU's memory that is not
    mapped here, faults.  Torch tensors say where they live, so refuse them here; other
    tensor-likes (the reference's own Tensor class) carry no device and pass."""
    is_cuda = getattr(t, "is_cuda", None)
    if is_cuda is None or _validate_only_depth > 0:
        return
    if not is_cuda:
        raise ValueError("expected a CUDA tensor, got one in host memory")
    import torch

    cur = torch.cuda.current_device()
    if t.device.index is not None and t.device.index != cur:
        raise ValueError(f"tensor lives on cuda:{t.device.index} but the current device is cuda:{cur}; "
                         "make its device current (torch.cuda.device) before the call")


def as_tensor(t) -> G4bTensor:
    """Packs a tensor-like (or None) into the C view; strides are in elements."""
    out = G4bTensor()
    if t is None:
        out.ptr = None
        out.ndim = 0
        return out
    if not (hasattr(t, "shape") and hasattr(t, "stride") and hasattr(t, "dtype") and hasattr(t, "data_ptr")):
        raise TypeError(f"expected a tensor-like with shape/stride/dtype/data_ptr, got {type(t).__name__}")
    _check_device(t)
    shape = list(t.shape)
    if len(shape) > 5:
        raise ValueError("tensors of rank > 5 are not supported")
    strides = _strides(t)
    out.ptr = int(t.data_ptr())
    for i, (n, s) in enumerate(zip(shape, strides)):
        out.shape[i] = int(n)
        out.stride[i] = int(s)
    out.ndim = len(shape)
    out.dtype = dtype_code(t.dtype)
    return out


def current_stream(stream=None) -> int:
    """Raw cudaStream_t: an int, an object with .cuda_stream, or torch's current stream."""
    if stream is None:
        import torch

        return int(torch.cuda.current_stream().cuda_stream)
    if isinstance(stream, int):
        return stream
    for attr in ("cuda_stream", "handle"):
        if hasattr(stream, attr):
            return int(getattr(stream, attr))
    raise TypeError(f"cannot take a CUDA stream from {stream!r}")


_VALUE_ERRORS = {-1, -2, -3, -4, -7}


def check(rc: int) -> None:
    """Maps a G4B_ERR_* code to ValueError (bad arguments) or RuntimeError (CUDA / device)."""
    if rc == 0 or rc == 1:      # 1 = G4B_VALIDATED (validate-only mode)
        return
    msg = load().g4b_last_error_string().decode("utf-8", "replace")
    if rc in _VALUE_ERRORS:
        raise ValueError(msg)
    raise RuntimeError(f"libg4b_attn error {rc}: {msg}")


def device_status(stream=None) -> int:
    """Synchronises the stream and returns (and clears) the device status word."""
    out = ctypes.c_int32(0)
    rc = load().g4b_device_status(ctypes.c_void_p(current_stream(stream)), ctypes.byref(out))
    if rc != -6:                # G4B_ERR_DEVICE_WAIT only says that the word was not zero
        check(rc)
    return int(out.value)
