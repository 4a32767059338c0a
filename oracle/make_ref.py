"""Copies the reference's own files for this path into git-ignored folders, so that they travel
to a GPU box with the repository snapshot while staying out of its history.

    python oracle/make_ref.py            # needs the reference checkout

TEST / BENCHMARK INFRASTRUCTURE ONLY; the product never reads these folders.

  oracle/_ref/scripts/reference_impl.py, oracle/_ref/g4b/gguf.py
      the reference's torch implementation of attention (LayerKVCache) and the one module it
      imports; oracle/ref_loader.py loads them, bench.py's reference arm times them
  baseline/_ref/g4b/kernels/fa2.py, baseline/_ref/g4b/kernels/utils.py
      the reference's Triton attention kernel and its launcher; baseline/triton_reference.py
      runs them on the GPU beside this library's kernels

The checkout is looked for in $G4B_REFERENCE_ROOT, then in a folder named ``reference`` beside
the repository.  Nothing is modified: the files are byte copies.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]

COPIES = [
    ("scripts/reference_impl.py", "oracle/_ref/scripts/reference_impl.py"),
    ("g4b/gguf.py", "oracle/_ref/g4b/gguf.py"),
    ("g4b/kernels/fa2.py", "baseline/_ref/g4b/kernels/fa2.py"),
    ("g4b/kernels/utils.py", "baseline/_ref/g4b/kernels/utils.py"),
]


def reference_checkout() -> Path | None:
    cands = [os.environ.get("G4B_REFERENCE_ROOT"), str(ROOT.parent / "reference")]
    for c in cands:
        if c and (Path(c) / "scripts" / "reference_impl.py").exists():
            return Path(c)
    return None


def make(verbose: bool = False) -> bool:
    """Returns True if the copies exist afterwards (made now or earlier)."""
    src_root = reference_checkout()
    if src_root is None:
        return all((ROOT / dst).exists() for _, dst in COPIES)
    for src, dst in COPIES:
        d = ROOT / dst
        d.parent.mkdir(parents=True, exist_ok=True)
        s = src_root / src
        if not d.exists() or d.read_bytes() != s.read_bytes():
            shutil.copyfile(s, d)
            if verbose:
                print(f"{s} -> {d}")
    return True


if __name__ == "__main__":
    ok = make(verbose=True)
    print("reference files in place" if ok else "reference checkout not found", file=sys.stderr)
    sys.exit(0 if ok else 1)
