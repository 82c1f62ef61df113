"""The reference's own callers, unmodified, on this library — and beside the reference's own kernels.

The staged tree baseline/_ref (baseline/stage_reference.py; ignored by version control, absent
means skip) holds the reference's Python and CUDA headers as they are.  tests/reference_runner.py
runs a job in a fresh process with `cuda_primitives` / `kquant_cuda` bound either to this library
(verinf_b200.shim) or to the reference's own JIT-built extension:

  * prover/tests/test_cuda_primitives.py:75-453 (25 acceptance tests, production geometry, ends in
    test_commit_phase_integration), prover/tests/test_persistent_weights.py:33-80 (core.commit_weights
    determinism under the fixed MASTER_SEED) and layergkr/tests/test_gpu.py:34-115 (GPU == CPU backend
    gates) must pass on the shim;
  * core.commit_weights (prover/core.py:874-910), encode_messages / hash_columns_streamed /
    merkle_build_blake3 at ELL=8192, K=16384, N=65536, and layergkr's sumcheck must give the same
    bytes on both backends (the reference's kernels are the second, independent witness).
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"
OUT = ROOT / "gpurun_out"

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (REF / "prover" / "core.py").exists(),
                                 reason="baseline/_ref not staged (python baseline/stage_reference.py)")]

_cache = {}


def run_job(backend: str, job: str, timeout: int = 900) -> dict:
    key = (backend, job)
    if key in _cache:
        return _cache[key]
    env = dict(os.environ)
    env.setdefault("TORCH_EXTENSIONS_DIR", str(ROOT / "build" / "torch_extensions"))   # the reference's JIT cache
    env.setdefault("MAX_JOBS", "8")
    p = subprocess.run([sys.executable, str(ROOT / "tests" / "reference_runner.py"), "--backend", backend, "--job", job],
                       capture_output=True, text=True, timeout=timeout, env=env, cwd=str(ROOT))
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    res = json.loads(lines[-1]) if lines else {"error": f"no result (rc {p.returncode}): {p.stderr[-2000:]}"}
    res["rc"] = p.returncode
    try:
        OUT.mkdir(exist_ok=True)
        (OUT / f"refrun_{backend.replace('+', '_')}_{job.replace(':', '_')}.json").write_text(json.dumps(res, indent=1))
    except OSError:
        pass
    _cache[key] = res
    return res


def reference_or_skip(job: str) -> dict:
    """The job on the reference's own kernels; skip (with its message) if they cannot be built here."""
    res = run_job("reference", job, timeout=1500)
    if "error" in res:
        pytest.skip("reference kernels unavailable on this machine: " + res["error"][-400:])
    assert res["cuda_primitives_file"].startswith("baseline/_ref/"), res["cuda_primitives_file"]
    return res


def shim(job: str, backend: str = "shim") -> dict:
    res = run_job(backend, job)
    assert "error" not in res, res["error"]
    assert res["cuda_primitives_file"] == "verinf_b200/cuda_primitives.py"
    return res


@pytest.mark.parametrize("module,min_tests", [("test_cuda_primitives", 25), ("test_persistent_weights", 3),
                                              ("test_gpu", 6)])
def test_reference_test_module_passes_on_shim(module, min_tests):
    res = shim(f"tests:{module}")
    assert not res["failed"], "\n".join(f"{k}:\n{v}" for k, v in res["failed"].items())
    assert len(res["passed"]) >= min_tests, res["passed"]


def test_layergkr_gates_pass_with_fused_routines():
    res = shim("tests:test_gpu", backend="shim+layergkr")
    assert not res["failed"], "\n".join(f"{k}:\n{v}" for k, v in res["failed"].items())
    assert len(res["passed"]) >= 6


def test_commit_weights_root_equals_reference_kernels():
    ours = shim("commit_weights")
    ref = reference_or_skip("commit_weights")
    for k in ("m_w", "root", "levels", "nodes", "levels_sha256"):
        assert ours[k] == ref[k], (k, ours[k], ref[k])


def test_production_geometry_kernels_equal_reference_kernels():
    ours = shim("kernels")
    ref = reference_or_skip("kernels")
    for k in ("polys_sha256", "codes_sha256", "leaves_sha256", "root", "n_levels", "ntt64x65536_sha256"):
        assert ours[k] == ref[k], (k, ours[k], ref[k])


def test_sumcheck_transcript_equals_reference_kernels():
    ours = shim("sumcheck")
    fused = shim("sumcheck", backend="shim+layergkr")
    assert ours["transcript_sha256"] == fused["transcript_sha256"] and ours["claim"] == fused["claim"]
    ref = reference_or_skip("sumcheck")
    assert ours["transcript_sha256"] == ref["transcript_sha256"] and ours["claim"] == ref["claim"]
