"""Multi-GPU (needs >= 2 visible GPUs, otherwise skipped): one process per GPU over NCCL.
Sharded single-tree commit and sharded sumcheck against the single-GPU results."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

WORKER = r'''
import os, sys
sys.path.insert(0, os.environ["VI_ROOT"])
import numpy as np, torch, torch.distributed as dist
from verinf_b200 import distributed as D, cuda_primitives as cp, layergkr_gpu as lg
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=dev)
P = cp.P
rng = np.random.default_rng(5)
def t64(a): return torch.from_numpy(np.ascontiguousarray(a).view(np.int64)).to(dev).view(torch.uint64)
total, ell, k, n = 2048 + 300, 1000, 1024, 4096
msg = rng.integers(0, P, size=(total, ell), dtype=np.uint64)
r0, r1 = D.split_rows(total, world)[rank]
root, levels, codes = D.commit_rows_sharded(t64(msg[r0:r1]), total, D.CudaBackend(k, n))
want_root, _, _ = cp.commit_rows(t64(msg), k, n)
assert torch.equal(root, want_root), "sharded root differs"
logn = 14
tabs = rng.integers(0, P, size=(3, 1 << logn), dtype=np.uint64)
coins = [int(c) for c in rng.integers(0, P, size=logn, dtype=np.uint64)]
terms = [(1, [0, 1, 2])]
full = lg.SumcheckProblem(t64(tabs), terms)
want_claim = full.claim(); want = []; r = None
for i in range(logn):
    want.append(full.round(r)); r = coins[i]
local = lg.SumcheckProblem(D.shard_table(t64(tabs), rank, world), terms)
claim, polys, chals = D.prove_terms_sharded(local, lambda t: lg.SumcheckProblem(t.contiguous(), terms),
                                            lambda i: coins[i], logn, dev)
assert claim == want_claim and [[y for _, y in rp] for rp in polys] == want and chals == coins
dist.barrier(); torch.cuda.synchronize()
if rank == 0: print("MULTI_OK", world)
dist.destroy_process_group()
'''


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_commit_and_sumcheck_nccl(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, VI_ROOT=str(ROOT), NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), str(script)],
                         env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and f"MULTI_OK {world}" in out.stdout, out.stdout[-2000:] + out.stderr[-4000:]
