"""Runs the reference's own Triton attention kernel on the GPU, beside this library's kernels.

BENCHMARK INFRASTRUCTURE ONLY: nothing in g4b_b200/ imports this file.

The kernel sources are the byte copies that oracle/make_ref.py leaves in baseline/_ref/
(g4b/kernels/fa2.py and its launcher g4b/kernels/utils.py, unmodified).  The reference engine
feeds them its own tensor class on a cuda.core stream; its launcher also takes any object with
shape / stride / dtype / data_ptr (g4b/kernels/utils.py:51-60,113-122: "to allow torch Tensors
as well for testing"), which is how its comparison script drives the kernel
(tests/compare_scripts/test_fa2.py:300-343) and how this file does.  What the two modules
import from the rest of the engine is stood in for here:

  g4b.tensor.Tensor   an empty class (only used in isinstance checks and annotations)
  g4b.device          device.create_event / stream.record / stream.sync over torch events on
                      torch's current stream (the autotuner's timer, utils.py:151-189, uses them)
  cuda.core           EventOptions, a plain record (the package is not installed here)

The reference has no softmax scale (fa2.py:89): q is scaled by the caller.  Its kernel needs a
ring cache [B, G, T, D], so paged benchmark inputs are laid out as rings for it.

    python baseline/triton_reference.py [--tuned] [--case NAME ...]

prints one JSON line: per case the time per launch, TFLOP/s or GB/s, the block sizes the
reference picked, the parity of its output against the CPU oracle on sampled rows, and the
time of this library's flash_attention on the very same tensors.
Without --tuned the reference's G4B_SKIP_TUNING=1 mode is used (its hand-picked production
configurations, fa2.py:152-158); with --tuned its whole autotune space is searched first;
--force M,N,SPLITS,WARPS,STAGES pins one configuration through the reference's own
G4B_FA_FORCE_CONFIG switch (fa2.py:147-149), for tile shapes its autotuner would have to find.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import time
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

H, G, D = 8, 2, 256
SCALE = 1.0 / 16.0


def available() -> bool:
    return (REF / "g4b" / "kernels" / "fa2.py").exists()


def load_reference_fa2(skip_tuning: bool = True, force: str | None = None):
    """Imports baseline/_ref/g4b/kernels/fa2.py with the stand-ins described above."""
    import torch

    if force:
        os.environ["G4B_FA_FORCE_CONFIG"] = force
    else:
        os.environ.pop("G4B_FA_FORCE_CONFIG", None)

    if not available():
        raise RuntimeError("baseline/_ref is empty: run `python oracle/make_ref.py` where the reference checkout is")
    if skip_tuning:
        os.environ["G4B_SKIP_TUNING"] = "1"
    else:
        os.environ.pop("G4B_SKIP_TUNING", None)
    for name in [m for m in sys.modules if m == "g4b" or m.startswith("g4b.")]:
        del sys.modules[name]

    pkg = types.ModuleType("g4b")
    pkg.__path__ = [str(REF / "g4b")]
    tensor_mod = types.ModuleType("g4b.tensor")

    class Tensor:  # stands in for g4b/tensor.py's class in isinstance checks
        pass

    tensor_mod.Tensor = Tensor

    class _Event:
        def __init__(self):
            self.ev = torch.cuda.Event(enable_timing=True)

        def sync(self):
            self.ev.synchronize()

        def __sub__(self, other):          # end - start -> milliseconds
            return other.ev.elapsed_time(self.ev)

    class _Device:
        def create_event(self, options=None):
            return _Event()

    class _Stream:
        def record(self, event):
            event.ev.record(torch.cuda.current_stream())

        def sync(self):
            torch.cuda.current_stream().synchronize()

    device_mod = types.ModuleType("g4b.device")
    device_mod.device, device_mod.stream = _Device(), _Stream()
    kernels_pkg = types.ModuleType("g4b.kernels")
    kernels_pkg.__path__ = [str(REF / "g4b" / "kernels")]
    pkg.tensor, pkg.device, pkg.kernels = tensor_mod, device_mod, kernels_pkg
    sys.modules.update({"g4b": pkg, "g4b.tensor": tensor_mod, "g4b.device": device_mod, "g4b.kernels": kernels_pkg})
    try:
        importlib.import_module("cuda.core")
    except Exception:
        import cuda

        core = types.ModuleType("cuda.core")

        class EventOptions:
            def __init__(self, **kw):
                self.__dict__.update(kw)

        core.EventOptions = EventOptions
        sys.modules["cuda.core"] = core
        cuda.core = core
    return importlib.import_module("g4b.kernels.fa2")


def _time_launches(fn, reps: int) -> float:
    import torch

    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def _sampled_parity(o, q, k_ring, v_ring, time_sizes, ctx_window, rows, what):
    """o / q [B,H,Tq,D] on the GPU; checks slot 0 (and the last slot) at the given query rows
    against the oracle, tolerance |a-b| <= 2e-3 + 1e-2 |b|."""
    import torch

    from oracle import attention_oracle as orc

    worst = 0.0
    B, _, Tq, _ = q.shape
    for b in sorted({0, B - 1}):
        t = int(time_sizes[b])
        k = orc.unroll_ring(k_ring[b].float().cpu(), t, ctx_window)
        v = orc.unroll_ring(v_ring[b].float().cpu(), t, ctx_window)
        window = k.shape[1]
        for r in rows:
            r = min(r, Tq - 1)
            pos = window - Tq + r
            want = orc.attention_core(q[b, :, r:r + 1].float().cpu(), k[:, :pos + 1], v[:, :pos + 1], scale=1.0)
            got = o[b, :, r:r + 1].float().cpu()
            err = (got - want).abs() - (2e-3 + 1e-2 * want.abs())
            worst = max(worst, float(err.max()))
    return ("ok" if worst <= 0 else f"{what}: exceeds tolerance by {worst:.3e}")


def run_case(fa2, name: str, dev, reps: int):
    import torch

    from g4b_b200.kernels import fa2 as our_fa2

    gen = torch.Generator(device=dev).manual_seed(17)
    rnd = lambda *s, dt: torch.randn(*s, generator=gen, device=dev, dtype=torch.float32).to(dt)
    picked = {}
    os.environ["G4B_FA_PRINT_CONFIG"] = ""
    if name == "prefill_causal":          # benchmark configuration 2
        B, S, dt = 4, 8192, torch.bfloat16
        q = (rnd(B, S, H, D, dt=torch.float32) * SCALE).to(dt).permute(0, 2, 1, 3)
        k, v = rnd(B, G, S, D, dt=dt), rnd(B, G, S, D, dt=dt)
        o = torch.zeros(B, S, H, D, device=dev, dtype=dt).permute(0, 2, 1, 3)
        t = torch.full((B,), S, dtype=torch.int32, device=dev)
        ph = torch.full((B,), fa2.PHASE_PREFILL, dtype=torch.uint8, device=dev)
        fn = lambda: fa2.flash_attention(q, k, v, o, t, ph, S, fa2.PHASE_PREFILL)
        o2 = torch.zeros(B, S, H, D, device=dev, dtype=dt).permute(0, 2, 1, 3)
        ours = lambda: our_fa2.flash_attention(q, k, v, o2, t, ph, S, our_fa2.PHASE_PREFILL)
        work, unit, div = 4.0 * B * H * D * (S * (S + 1) // 2), "TFLOP/s", 1e12
        rows, ctx = (0, 4097, S - 1), S
    elif name == "decode_ring":           # benchmark configuration 4, laid out as rings
        B, T, dt = 64, 32768, torch.float16
        lens = torch.randint(1024, 32769, (B,), generator=torch.Generator().manual_seed(3), dtype=torch.int64)
        q = (rnd(B, 1, H, D, dt=torch.float32) * SCALE).to(dt).permute(0, 2, 1, 3)
        k, v = rnd(B, G, T, D, dt=dt), rnd(B, G, T, D, dt=dt)
        o = torch.zeros(B, 1, H, D, device=dev, dtype=dt).permute(0, 2, 1, 3)
        t = lens.to(torch.int32).to(dev)
        ph = torch.full((B,), fa2.PHASE_DECODE, dtype=torch.uint8, device=dev)
        S_ = 16
        po = torch.empty(S_, B, H, 1, D, device=dev, dtype=dt)       # the engine's partial_o is f16 (gemma4e.py:819-821)
        pl, pm = torch.empty(S_, B, H, 1, device=dev), torch.empty(S_, B, H, 1, device=dev)
        fn = lambda: fa2.flash_attention(q, k, v, o, t, ph, T, fa2.PHASE_DECODE, po, pl, pm)
        o2 = torch.zeros(B, 1, H, D, device=dev, dtype=dt).permute(0, 2, 1, 3)
        ours = lambda: our_fa2.flash_attention(q, k, v, o2, t, ph, T, our_fa2.PHASE_DECODE, po, pl, pm)
        work, unit, div = float(lens.sum()) * G * D * 2 * 2, "GB/s", 1e9
        rows, ctx = (0,), T
    else:
        raise ValueError(name)
    t0 = time.perf_counter()
    fn()                                   # compiles, and tunes when tuning is on
    torch.cuda.synchronize()
    first_call_s = time.perf_counter() - t0
    ms = _time_launches(fn, reps)
    kern = fa2._attn_kernel
    best = getattr(kern, "best_config", None)
    if best is not None:
        picked = {**best.kwargs, "num_warps": best.num_warps, "num_stages": best.num_stages}
    parity = _sampled_parity(o, q, k, v, t.cpu(), ctx, rows, name)
    ms_ours = _time_launches(ours, max(reps, 10))
    parity_ours = _sampled_parity(o2, q, k, v, t.cpu(), ctx, rows, name)
    return {"case": name, "ms_per_launch": round(ms, 4), "value": round(work / (ms * 1e-3) / div, 3), "unit": unit,
            "picked": picked, "first_call_s": round(first_call_s, 1), "parity_vs_oracle": parity,
            "dtype": str(q.dtype).replace("torch.", ""),
            "this_library_same_tensors": {"ms_per_launch": round(ms_ours, 4),
                                          "value": round(work / (ms_ours * 1e-3) / div, 3),
                                          "parity_vs_oracle": parity_ours, "speedup": round(ms / ms_ours, 2)}}


def run(cases, tuned: bool, reps: int = 5, force: str | None = None):
    """Returns {"skip_tuning": ..., "cases": [...]} or {"unavailable": reason}."""
    import torch

    if not available():
        return {"unavailable": "baseline/_ref is empty (oracle/make_ref.py has not run where the reference checkout is)"}
    try:
        import triton

        fa2 = load_reference_fa2(skip_tuning=not tuned, force=force)
    except Exception as exc:
        return {"unavailable": f"import of the reference kernel failed: {type(exc).__name__}: {str(exc)[:300]}"}
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {"triton": triton.__version__, "skip_tuning": not tuned, "forced_config": force, "cases": []}
    for name in cases:
        try:
            out["cases"].append(run_case(fa2, name, dev, reps))
        except Exception as exc:
            msg = f"{type(exc).__name__}: {str(exc)[:400]}"
            out["cases"].append({"case": name, "unavailable": msg})
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tuned", action="store_true", help="search the reference's whole autotune space first")
    ap.add_argument("--case", action="append", choices=["prefill_causal", "decode_ring"])
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--force", help="Q_BLOCKSIZE_T,KV_BLOCKSIZE_T,NUM_KV_SPLITS,num_warps,num_stages")
    args = ap.parse_args()
    print(json.dumps(run(args.case or ["prefill_causal", "decode_ring"], args.tuned, args.reps, args.force)))


if __name__ == "__main__":
    main()
