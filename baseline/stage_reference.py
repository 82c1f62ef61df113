"""Stages the reference's own Python callers and CUDA headers for runs on a GPU machine.

The reference tree is read-only and exists only where this project is built, so the files its
callers need (prover/*.py, prover/ref, prover/kernels, prover/tests, demo, and layergkr with its tests) are copied unmodified into baseline/_ref/, which version
control ignores.  tests/test_reference_callers.py and `bench.py --extra` then run the
reference's own call stacks from there -- once on this library through verinf_b200.shim, once
on the reference's own JIT-built kernels -- and skip when the directory is absent.

    python baseline/stage_reference.py [/path/to/reference]
"""
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
DEFAULT_SRC = Path("/root/reference")

# (sub-directory, glob) pairs copied; nothing outside these is needed by the staged call stacks
WANTED = [
    ("prover", "*.py"),
    ("prover/ref", "*.py"),
    ("prover/kernels", "*.cuh"),
    ("layergkr", "*.py"),
    ("layergkr/tests", "*.py"),
    ("prover/tests", "*.py"),
    ("prover/tests/vectors", "*.json"),
    ("demo", "*.py"),
    ("demo", "*.txt"),
]
WANTED_FILES = [
    "LICENSE",
]


def stage(src: Path = DEFAULT_SRC, dest: Path = DEST) -> bool:
    """Copies the files; returns False (and leaves dest alone) when the reference is not there."""
    src = Path(src)
    if not (src / "prover" / "cuda_primitives.py").exists():
        return False
    n = 0
    for sub, pat in WANTED:
        for f in sorted((src / sub).glob(pat)):
            out = dest / sub / f.name
            out.parent.mkdir(parents=True, exist_ok=True)
            if not out.exists() or out.read_bytes() != f.read_bytes():
                shutil.copy2(f, out)
            n += 1
    for rel in WANTED_FILES:
        f = src / rel
        if f.exists():
            out = dest / rel
            out.parent.mkdir(parents=True, exist_ok=True)
            if not out.exists() or out.read_bytes() != f.read_bytes():
                shutil.copy2(f, out)
            n += 1
    (dest / "STAGED_FROM").write_text(f"{src}\n{n} files, unmodified\n")
    return True


if __name__ == "__main__":
    ok = stage(Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_SRC)
    print("staged into", DEST if ok else "(reference not found; nothing staged)")
