"""Runs the reference's own call stacks in a fresh process, on one of two backends.

    python tests/reference_runner.py --backend shim|shim+layergkr|reference --job JOB

The staged reference tree (baseline/_ref, see baseline/stage_reference.py) is put on sys.path
unmodified.  With `--backend shim` the modules `cuda_primitives` / `kquant_cuda` are this
library's (verinf_b200.shim.install()); with `--backend reference` they are the reference's
own, JIT-built from its CUDA headers by its own `load_inline` call.  Module names collide, so
each backend needs its own process.  `shim+layergkr` additionally swaps this package's fused
encode / commit / sumcheck routines into the reference's `layergkr.gpu` module
(verinf_b200.shim.install_layergkr()).  The last stdout line is a JSON object.

Jobs
  tests:<module>   import a reference test module (any of prover/tests/*.py, layergkr/tests/*.py, e.g.
                   test_cuda_primitives, test_persistent_weights, test_claims, test_gpu) and call
                   every test_* function, as the reference's run_tests.py does
  proofs:<module>  the same, for modules whose tests end in the Rust verifier: a stand-in records the
                   SHA-256 of every dumped proof file instead (see job_proofs)
  demo:<name>      demo/demo_<name>.py (llama7b): a whole transformer block proved and dumped; digest of the file
  script:<name>    a reference test script that runs at import (difftest_lde_skip): the digests it prints
  kquant           kquant_cuda.kquant_to_field against gguf-py's dequantize -> quantize_to_field on seeded blocks
  commit_weights   core.commit_weights (prover/core.py:874-910) of a small seeded tape at the
                   production geometry: root and a digest of every Merkle level
  kernels          encode_messages + hash_columns_streamed + merkle_build_blake3 at
                   ELL=8192, K=16384, N=65536 on 1024 seeded rows: digests of the outputs and
                   CUDA-event times
  sumcheck         layergkr sumcheck.prove_terms through gpu.prove_terms_gpu on seeded tables
"""
import argparse
import hashlib
import importlib
import json
import sys
import time
import traceback
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"
P = (1 << 64) - (1 << 32) + 1


def setup(backend: str) -> None:
    if not (REF / "prover" / "core.py").exists():
        raise SystemExit("baseline/_ref is not staged (python baseline/stage_reference.py)")
    sys.path.insert(0, str(ROOT))
    if backend.startswith("shim"):
        from verinf_b200 import shim
        shim.install()
    # the reference's own entry points push prover/ to sys.path[0] themselves; repeat it for direct imports
    sys.path.insert(0, str(REF))
    sys.path.insert(0, str(REF / "prover"))
    import torch  # noqa: F401
    import _uint64_compat  # noqa: F401  (the reference imports it before any prover op, demo/demo_llama7b.py:74)
    if backend == "shim+layergkr":
        shim.install_layergkr()


def backend_identity() -> dict:
    import cuda_primitives as cp
    return {"cuda_primitives_file": str(Path(cp.__file__).resolve().relative_to(ROOT))}


def job_tests(modname: str) -> dict:
    path = next((d for d in (REF / "prover" / "tests", REF / "layergkr" / "tests") if (d / f"{modname}.py").exists()), None)
    if path is None:
        raise SystemExit(f"no staged reference test module {modname}")
    sys.path.insert(0, str(path))
    mod = importlib.import_module(modname)
    passed, failed = [], {}
    for name in [n for n in dir(mod) if n.startswith("test_") and callable(getattr(mod, n))]:
        t0 = time.time()
        try:
            getattr(mod, name)()
            passed.append([name, round(time.time() - t0, 3)])
        except Exception:  # noqa: BLE001  (report every failure, keep going)
            failed[name] = traceback.format_exc()[-1500:]
    return {"module": modname, "passed": passed, "failed": failed}


def job_proofs(modname: str) -> dict:
    """Every test_* of a reference test module that proves and then hands the dumped proof to the Rust
    verifier (prover/tests/_rust_verify.py:51-77).  No Rust toolchain exists on these machines, so
    LIGERO_VERIFY_PROOF points at a stand-in that records the SHA-256 of each dumped proof file and its
    policy arguments and answers "UNVERIFIED" (never ACCEPT): honest-case tests then stop at their
    `assert acc`, which is recorded as such, and anything raised before the verifier is reached is a
    real failure.  The per-test digest lists of two backends are what gets compared; with
    VERINF_PROOF_KEEP=<dir> the stand-in also keeps a copy of every proof file there."""
    import os
    import stat
    import tempfile
    tmp = Path(tempfile.mkdtemp(prefix="verinf_proofs_"))
    log = tmp / "digests.txt"
    stub = tmp / "verify_proof_stub.sh"
    stub.write_text('#!/bin/sh\n'
                    'printf "%s %s %s\\n" "$(sha256sum "$1" | cut -d" " -f1)" "$2" "$3" >> "' + str(log) + '"\n'
                    'if [ -n "$VERINF_PROOF_KEEP" ]; then mkdir -p "$VERINF_PROOF_KEEP"; '
                    'cp "$1" "$VERINF_PROOF_KEEP/$(wc -l < "' + str(log) + '").json"; fi\n'
                    'echo "rust_verify: UNVERIFIED (stand-in: no Rust verifier on this machine, digest recorded)"\n'
                    'exit 3\n')
    stub.chmod(stub.stat().st_mode | stat.S_IXUSR)
    os.environ["LIGERO_VERIFY_PROOF"] = str(stub)
    _fix_secrets()
    out = job_tests_with(modname, log)
    return out


def _fix_secrets() -> None:
    """The production prover pads and blinds under a fresh secret per proof (core.new_zk_seed ->
    secrets.token_bytes, prover/core.py:3265-3275), so two runs never dump the same bytes.  For a
    comparison the source of those secrets is replaced by a counter-keyed hash, the same in both processes."""
    import secrets
    ctr = [0]

    def fixed_token_bytes(n=32):
        ctr[0] += 1
        return hashlib.sha256(b"verinf_b200 proofs job " + str(ctr[0]).encode()).digest()[:n]
    secrets.token_bytes = fixed_token_bytes


def job_demo(name: str) -> dict:
    """demo/demo_<name>.py main() without a checkpoint: one transformer block of the demo's architecture
    (demo_llama7b: d = 4096, d_ff = 11008, SEQ = 2 at ELL=8192/K=16384/N=65536; RmsNorm, Q/K/V/O and FFN
    matmuls, RoPE, softmax, SiLU, Hadamard, residual adds) with seeded random weights, proved by tape.prove
    and dumped by the reference's proof writer; digest and size of the dumped file.  LIGERO_T_QUERIES
    (default here 4) sets the number of opened columns, which only sizes the dump."""
    import os
    import tempfile
    os.environ.setdefault("LIGERO_T_QUERIES", "4")
    import torch
    _fix_secrets()
    torch.manual_seed(20240611)
    torch.cuda.manual_seed_all(20240611)
    sys.path.insert(0, str(REF / "demo"))
    demo = importlib.import_module(f"demo_{name}")
    fd, path = tempfile.mkstemp(suffix=".json")
    os.close(fd)
    import contextlib
    import io
    import re
    torch.cuda.synchronize()
    t0 = time.time()
    log = io.StringIO()
    try:
        with contextlib.redirect_stdout(log):
            demo.main(dump_proof=path, with_lm_head=False, engine=True)
        torch.cuda.synchronize()
        dt = time.time() - t0
        h, nbytes = hashlib.sha256(), 0
        with open(path, "rb") as f:
            for blk in iter(lambda: f.read(1 << 24), b""):
                h.update(blk)
                nbytes += len(blk)
    finally:
        os.unlink(path)
    m = re.findall(r"prove:\s+([0-9.]+)s", log.getvalue())       # the demo's own timer around tape.prove
    return {"demo": name, "proof_sha256": h.hexdigest(), "proof_bytes": nbytes, "s": dt,
            "prove_s": float(m[-1]) if m else None, "peak_gb": torch.cuda.max_memory_allocated() / 1e9}


def job_script(name: str) -> dict:
    """A reference test script that runs at import (prover/tests/difftest_lde_skip.py: one tape at ELL = K = 8,
    N = 32 proved with the codeword pass skipped where unread and forced, both proofs dumped and hashed):
    executed as __main__ with its output captured; the SHA-256 values it prints are returned in order."""
    import contextlib
    import io
    import re
    import runpy
    _fix_secrets()
    sys.path.insert(0, str(REF / "prover" / "tests"))
    log = io.StringIO()
    code = None
    with contextlib.redirect_stdout(log):
        try:
            runpy.run_path(str(REF / "prover" / "tests" / f"{name}.py"), run_name="__main__")
        except SystemExit as e:         # the script ends in `raise SystemExit(0 if identical else 1)`
            code = e.code
    text = log.getvalue()
    return {"script": name, "exit": code, "digests": re.findall(r"\b[0-9a-f]{64}\b", text),
            "lines": len(text.splitlines())}


def job_kquant() -> dict:
    """The gate of prover/tests/test_kquant_kernel.py:31-62 on seeded synthetic super-blocks (that test needs a
    real GGUF file): kquant_to_field of Q4_K / Q5_K / Q6_K bytes against gguf.quants.dequantize ->
    loader.quantize_to_field, 4096 blocks per type, scales drawn as finite fp16 values of mixed magnitude."""
    import numpy as np
    import torch
    from gguf import GGMLQuantizationType
    from gguf.quants import dequantize
    from kquant_cuda import kquant_to_field
    from loader import quantize_to_field
    S = 1 << 12
    out = {}
    for qt, nbytes, scale_at in (("Q4_K", 144, (0, 2)), ("Q5_K", 176, (0, 2)), ("Q6_K", 210, (208,))):
        rng = np.random.default_rng(len(qt) * 1000 + nbytes)
        raw = rng.integers(0, 256, (4096, nbytes), dtype=np.uint8)
        for off in scale_at:                     # d / dmin: finite halves between 2^-14 and 2^2, either sign
            h = (rng.uniform(-1, 1, 4096) * np.exp2(rng.integers(-14, 3, 4096))).astype(np.float16)
            raw[:, off:off + 2] = h.view(np.uint8).reshape(4096, 2)
        ref = quantize_to_field(torch.from_numpy(dequantize(raw, GGMLQuantizationType[qt]).copy()), S).reshape(-1)
        got = kquant_to_field(torch.from_numpy(raw).cuda(), qt, S)
        out[qt] = {"equals_gguf_numpy": bool(torch.equal(ref.view(torch.int64), got.view(torch.int64))),
                   "sha256": _sha(got), "n": int(got.numel())}
    return {"kquant": out}


def job_tests_with(modname: str, log: Path) -> dict:
    path = next((d for d in (REF / "prover" / "tests", REF / "layergkr" / "tests") if (d / f"{modname}.py").exists()), None)
    if path is None:
        raise SystemExit(f"no staged reference test module {modname}")
    sys.path.insert(0, str(path))
    mod = importlib.import_module(modname)
    res = {}
    for name in sorted(n for n in dir(mod) if n.startswith("test_") and callable(getattr(mod, n))):
        before = log.read_text().splitlines() if log.exists() else []
        status = "passed"
        try:
            getattr(mod, name)()
        except AssertionError as e:
            status = "assert: " + str(e)[:160]
        except Exception:  # noqa: BLE001
            status = "error: " + traceback.format_exc()[-600:]
        after = log.read_text().splitlines() if log.exists() else []
        res[name] = {"status": status, "proofs": after[len(before):]}
    return {"module": modname, "tests": res}


def _sha(t) -> str:
    import torch
    if t.dtype == torch.uint64:
        t = t.view(torch.int64)
    return hashlib.sha256(t.contiguous().cpu().numpy().tobytes()).hexdigest()


def job_commit_weights() -> dict:
    import torch
    import core
    from tape import Tape
    cfg = core.LigeroConfig(ELL=8192, K_DEG=16384, N_LIG=65536, T_QUERIES=4)
    tape = Tape(cfg, lazy=True)
    g = torch.Generator().manual_seed(20240607)
    for name, n in (("W_a", 70000), ("W_b", 1200000), ("W_c", 3333)):
        data = torch.randint(0, 1 << 20, (n,), dtype=torch.int64, generator=g).to(torch.uint64).cuda()
        wt = tape.commit(name, data, (n,), persistent=True)
        tape.add(wt, wt)
    art, _, m_w = core.commit_weights(tape, cfg)
    h = hashlib.sha256()
    n_nodes = 0
    for lvl in art.levels:
        for node in lvl:
            h.update(bytes(node))
            n_nodes += 1
    return {"m_w": int(m_w), "root": bytes(art.root).hex(), "levels": len(art.levels), "nodes": n_nodes,
            "levels_sha256": h.hexdigest()}


def job_kernels() -> dict:
    import torch
    import core
    from cuda_primitives import hash_columns_streamed, merkle_build_blake3, ntt_forward_batched
    cfg = core.LigeroConfig(ELL=8192, K_DEG=16384, N_LIG=65536, T_QUERIES=4)
    m = 1024
    g = torch.Generator(device="cuda").manual_seed(99)
    msgs = torch.randint(0, 1 << 62, (m, cfg.ELL), generator=g, dtype=torch.int64, device="cuda").view(torch.uint64)
    seed = torch.arange(32, dtype=torch.uint8, device="cuda")

    def timed(fn, reps=3):
        best, out = None, None
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            out = fn()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b)
            best = ms if best is None else min(best, ms)
        return out, best

    (polys, codes), enc_ms = timed(lambda: core.encode_messages(msgs, cfg, master_seed=seed, row_offset=5))
    leaves, hash_ms = timed(lambda: hash_columns_streamed(codes))
    (root, levels), merkle_ms = timed(lambda: merkle_build_blake3(leaves))
    # a plain batched NTT at the codeword length, the reference's Bailey path
    x = msgs[:64].repeat(1, 8).contiguous()
    _, ntt_ms = timed(lambda: ntt_forward_batched(x))
    return {"rows": m, "ELL": cfg.ELL, "K": cfg.K_DEG, "N": cfg.N_LIG,
            "polys_sha256": _sha(polys), "codes_sha256": _sha(codes), "leaves_sha256": _sha(leaves),
            "root": bytes(root.cpu().tolist()).hex(), "n_levels": len(levels),
            "ntt64x65536_sha256": _sha(x),
            "encode_ms": enc_ms, "hash_ms": hash_ms, "merkle_ms": merkle_ms, "ntt64x65536_x3_ms": ntt_ms}


def job_sumcheck() -> dict:
    """layergkr.sumcheck.prove_terms above its device threshold (size * factors >= 2^16 routes to
    gpu.prove_terms_gpu, layergkr/sumcheck.py:170-181), bare and masked (`tape`, `mu0`)."""
    import random
    from layergkr import sumcheck
    from layergkr.transcript import Transcript
    r = random.Random(11)
    logn = 15
    n = 1 << logn
    tabs = [[r.randrange(P) for _ in range(n)] for _ in range(3)]
    tr = Transcript(b"runner/sumcheck")
    tr.absorb("seed", (7).to_bytes(8, "little"))
    coins = tr.coin("sc", logn)
    terms = [(1, [tabs[0], tabs[1], tabs[2]]), (P - 5, [tabs[1], tabs[2]])]
    assert sumcheck._sumcheck_gpu_ok(), "the reference's own GPU == CPU sumcheck gate failed on this backend"
    t0 = time.time()
    pf = sumcheck.prove_terms(terms, lambda i: coins[i])
    dt = time.time() - t0
    tape = sumcheck.MaskTape([r.randrange(P) for _ in range(3 * logn)])
    pm = sumcheck.prove_terms(terms, lambda i: coins[i], tape=tape, mu0=123456789)
    h = hashlib.sha256(repr((pf.claim, pf.round_polys, pf.challenges,
                             pm.claim, pm.round_polys, pm.challenges, pm.final_mask)).encode()).hexdigest()
    return {"n": n, "claim": int(pf.claim), "masked_claim": int(pm.claim), "transcript_sha256": h, "s": dt}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", choices=["shim", "shim+layergkr", "reference"], required=True)
    ap.add_argument("--job", required=True)
    a = ap.parse_args()
    setup(a.backend)
    out = {"backend": a.backend, "job": a.job}
    try:
        out.update(backend_identity())
        if a.job.startswith("tests:"):
            out.update(job_tests(a.job.split(":", 1)[1]))
        elif a.job.startswith("proofs:"):
            out.update(job_proofs(a.job.split(":", 1)[1]))
        elif a.job.startswith("demo:"):
            out.update(job_demo(a.job.split(":", 1)[1]))
        elif a.job.startswith("script:"):
            out.update(job_script(a.job.split(":", 1)[1]))
        elif a.job == "kquant":
            out.update(job_kquant())
        elif a.job == "commit_weights":
            out.update(job_commit_weights())
        elif a.job == "kernels":
            out.update(job_kernels())
        elif a.job == "sumcheck":
            out.update(job_sumcheck())
        else:
            raise SystemExit(f"unknown job {a.job}")
    except Exception:  # noqa: BLE001
        out["error"] = traceback.format_exc()[-3000:]
    print(json.dumps(out))


if __name__ == "__main__":
    main()
