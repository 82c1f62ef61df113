"""The reference's own callers, unmodified, on this library — and beside the reference's own kernels.

The staged tree baseline/_ref (baseline/stage_reference.py; ignored by version control, absent
means skip) holds the reference's Python and CUDA headers as they are.  tests/reference_runner.py
runs a job in a fresh process with `cuda_primitives` / `kquant_cuda` bound either to this library
(verinf_b200.shim) or to the reference's own JIT-built extension:

  * prover/tests/test_cuda_primitives.py:75-453 (25 acceptance tests, production geometry, ends in
    test_commit_phase_integration), prover/tests/test_persistent_weights.py:33-80 (core.commit_weights
    determinism under the fixed MASTER_SEED), layergkr/tests/test_gpu.py:34-115 (GPU == CPU backend
    gates) and the other test modules listed below must pass on the shim;
  * the prover tests that end in the Rust verifier (prover/tests/test_claims.py, test_routing_claim.py,
    test_fiat_shamir.py, ... through prover/tests/_rust_verify.py) are run with a stand-in that records the
    SHA-256 of every proof file the reference's own writer (prover/proof_dump.py) dumps: the flat test
    prover and the production streaming prover (tape.prove -> core.prove_streaming) must dump the same
    bytes on both backends, with the per-proof secrets fixed;
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
                                              ("test_gpu", 6), ("test_gather_rows", 9),
                                              ("test_iter_message_chunks", 15), ("test_opening_ledger", 6),
                                              ("test_pkt_range", 13), ("test_quad_eval_accumulator", 1)])
def test_reference_test_module_passes_on_shim(module, min_tests):
    res = shim(f"tests:{module}")
    assert not res["failed"], "\n".join(f"{k}:\n{v}" for k, v in res["failed"].items())
    assert len(res["passed"]) >= min_tests, res["passed"]


@pytest.mark.parametrize("module,min_tests", [("test_gpu", 6), ("test_rs", 4), ("test_sumcheck", 11), ("test_layer", 8),
                                              ("test_full_layer", 17), ("test_moe", 13), ("test_logup", 12),
                                              ("test_projection", 13)])
def test_layergkr_test_module_passes_with_fused_routines(module, min_tests):
    """layergkr's own tests with this package's encode / commit / sumcheck routines set on layergkr.gpu
    (shim.install_layergkr): the layer provers of full_layer.py, layer.py and moe.py reach them through
    rs.py and sumcheck.py; test_full_layer's gate batch has hundreds of tables in one sumcheck."""
    res = shim(f"tests:{module}", backend="shim+layergkr")
    assert not res["failed"], "\n".join(f"{k}:\n{v}" for k, v in res["failed"].items())
    assert len(res["passed"]) >= min_tests, res["passed"]


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


PROOF_MODULES = ["test_claims", "test_routing_claim", "test_fiat_shamir", "test_persistent_weights_link",
                 "test_persistent_weights_p3", "test_persistent_weights_p5", "test_phase3_block", "test_reveal",
                 "test_concat_claim", "test_rescale_claim", "test_routed_projected", "test_rmsnorm_bracket",
                 "test_shard_streaming", "test_moe_routed", "test_empty_root_sentinel"]


def test_dumped_proofs_byte_identical_to_reference_kernels():
    """Every proof the reference's prover tests dump for the Rust verifier (75 proofs: honest cases,
    cheating provers, Fiat-Shamir, persistent-weight linking, phase-3 blocks, routed MoE projections) has
    the same SHA-256 whether the primitives underneath are this library's or the reference's own kernels,
    and every test ends the same way on both (no Rust verifier here: honest cases stop at `assert acc`)."""
    from concurrent.futures import ThreadPoolExecutor
    reference_or_skip("kernels")                       # builds the reference's extension once, or skips
    jobs = [(b, f"proofs:{m}") for m in PROOF_MODULES for b in ("shim", "reference")]
    with ThreadPoolExecutor(max_workers=6) as pool:
        list(pool.map(lambda bj: run_job(bj[0], bj[1], timeout=1500), jobs))
    n_proofs, summary = 0, {}
    for m in PROOF_MODULES:
        ours, ref = shim(f"proofs:{m}"), reference_or_skip(f"proofs:{m}")
        assert ours["tests"].keys() == ref["tests"].keys() and ours["tests"], m
        for name, t in ours["tests"].items():
            r = ref["tests"][name]
            assert t["proofs"] == r["proofs"], (m, name, t["proofs"], r["proofs"])
            assert t["status"][:60] == r["status"][:60], (m, name, t["status"], r["status"])
            assert not t["status"].startswith("error"), (m, name, t["status"])
            n_proofs += len(t["proofs"])
        summary[m] = {"tests": len(ours["tests"]), "proofs": sum(len(t["proofs"]) for t in ours["tests"].values())}
    assert n_proofs >= 70, summary
    try:
        (OUT / "refrun_proofs_summary.json").write_text(json.dumps({"identical_proofs": n_proofs, "modules": summary}, indent=1))
    except OSError:
        pass


def test_llama7b_block_proof_byte_identical_to_reference_kernels():
    """demo/demo_llama7b.py, the reference's production driver, without a checkpoint: one Llama-2-7B-shaped
    block (d = 4096, d_ff = 11008, SEQ = 2, seeded random weights) at ELL=8192/K=16384/N=65536, committed and
    proved by the streaming prover and dumped by the reference's proof writer.  The 6 MB proof file has the
    same SHA-256 on this library and on the reference's own kernels."""
    from concurrent.futures import ThreadPoolExecutor
    reference_or_skip("kernels")
    with ThreadPoolExecutor(max_workers=2) as pool:
        list(pool.map(lambda b: run_job(b, "demo:llama7b", timeout=1500), ("shim", "reference")))
    ours, ref = shim("demo:llama7b"), reference_or_skip("demo:llama7b")
    assert ours["proof_bytes"] == ref["proof_bytes"] > 1 << 20
    assert ours["proof_sha256"] == ref["proof_sha256"]


def test_kquant_lift_equals_reference_kernel_and_gguf():
    """prover/tests/test_kquant_kernel.py's gate on synthetic super-blocks: both kernels equal
    gguf.quants.dequantize -> loader.quantize_to_field, and each other, for Q4_K, Q5_K, Q6_K."""
    ours, ref = shim("kquant"), reference_or_skip("kquant")
    for qt in ("Q4_K", "Q5_K", "Q6_K"):
        assert ours["kquant"][qt]["equals_gguf_numpy"] and ref["kquant"][qt]["equals_gguf_numpy"], qt
        assert ours["kquant"][qt]["sha256"] == ref["kquant"][qt]["sha256"], qt


def test_lde_skip_difftest_smallest_geometry():
    """prover/tests/difftest_lde_skip.py: a tape at ELL = K = 8, N = 32 (no pad slack, 8- and 32-point transforms)
    proved under a pinned ZK seed with and without the codeword pass of the q-polynomial round; the script's
    two proof digests must be equal to each other and to the ones the reference's kernels give."""
    ours, ref = shim("script:difftest_lde_skip"), reference_or_skip("script:difftest_lde_skip")
    assert ours["exit"] == 0 and len(ours["digests"]) == 2 and ours["digests"][0] == ours["digests"][1]
    assert ours["digests"] == ref["digests"]
