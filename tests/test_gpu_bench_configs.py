"""The benchmark's own configurations, pinned: `bench.py` at one GPU commits the large-batch
configuration (4096 x 2^16 -> 2^18), runs the 2^24 x 3 sumcheck with the seeded transcript's coins,
the fused K-quant lift + encode of the 11008 x 4096 weight and the 7B-layer commit + sumcheck, and
its CPU leg recomputes each of them with the oracle on the same data (whole-batch Merkle root, full
sumcheck transcript, first / last / 16 spread rows of the fused encode, the W_Q commitment and its
sumcheck).  This test runs that and requires every equality."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu


def test_bench_self_check_on_the_quoted_configurations():
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "2", "--warmup", "3", "--no-e2e"],
                       capture_output=True, text=True, timeout=1500, cwd=str(ROOT))
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    line = json.loads([ln for ln in p.stdout.splitlines() if ln.startswith("{")][-1])
    try:
        (ROOT / "gpurun_out").mkdir(exist_ok=True)
        (ROOT / "gpurun_out" / "bench_self_check.json").write_text(json.dumps(line, indent=1))
    except OSError:
        pass
    assert line.get("commit_root_equals_oracle") or line.get("commit_prefix_root_equals_oracle")
    assert line["sumcheck_transcript_equals_oracle"] is True
    assert line["kquant_rows_equal_oracle"] == {"Q4_K": True, "Q6_K": True}
    assert line["layer7b_W_Q_root_equals_oracle"] is True and line["layer7b_W_Q_sumcheck_equals_oracle"] is True
    assert all(r["bit_identical_to_unfused"] for r in line["kquant_fused_encode"])
    assert line["layer7b"]["sumcheck_claims_match_rho_Y_tau"] is True
    assert line["sharded_commit"]["root"] == line["config"]["root"]
    assert line["gpu_launches"] > 0 and line["roofline"]["frac"] > 0
