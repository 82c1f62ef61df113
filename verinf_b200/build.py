"""Build libverinf_b200.so (sm_100a) in-tree with nvcc.  `python -m verinf_b200.build`."""
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
SO = HERE / "libverinf_b200.so"
SOURCES = ["common.cu", "ntt.cu", "hash.cu", "field_ops.cu", "kquant.cu", "sumcheck.cu", "open.cu", "matmul_tc.cu", "matmul_umma.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def needs_build() -> bool:
    if not SO.exists():
        return True
    t = SO.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "verinf_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return SO
    objs = []
    procs = []
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    extra = os.environ.get("VERINF_NVCC_EXTRA", "").split()      # experiment switches, e.g. -DVGL_SHIFT_ALU
    for src in SOURCES:
        obj = CSRC / (src[:-3] + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)))
        objs.append(str(obj))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src} ---\n{out.decode(errors='replace')}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see messages above")
    subprocess.check_call([_nvcc(), "-shared", "-o", str(SO), *objs, "-Xcompiler", "-fPIC"], env=env)
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
