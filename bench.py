"""Benchmark of the commit hot path: RS-encoded Goldilocks elements per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

One step = one commit of the large-batch configuration (4096 rows x 2^16 uniform field
elements, blow-up 4 by coset NTT to 2^18 columns, BLAKE3 column leaves, Merkle root).
With N > 1 (launched by torchrun, one rank per GPU) every rank commits its own batch
of the same size — independent commits, no data-path collective; the 32-byte roots are
all-gathered — so the job is weak-scaled and `value` is the aggregate over all ranks.

`--impl reference` times the CPU restatement of the reference algorithm (the oracle,
OpenMP over all host threads) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

P = (1 << 64) - (1 << 32) + 1
METRIC = "RS-encoded Goldilocks elems/s"
UNIT = "elems/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--log-k", type=int, default=16)
    ap.add_argument("--blowup", type=int, default=4)
    ap.add_argument("--cpu-rows", type=int, default=0, help="rows of the CPU sample (0 = auto)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--sumcheck", action="store_true", help="also time the 2^24 degree-3 sumcheck")
    ap.add_argument("--extra", action="store_true",
                    help="also run the secondary workloads: fused K-quant lift+encode, 7B-layer commit+sumcheck")
    ap.add_argument("--micro", choices=["matmul", "fold", "sumcheck", "int_pipes"],
                    help="run only one secondary kernel (1024 x 2048 x 2048 matmul, the fold of 1024 row pairs "
                         "at K = 16384, or the 2^24 x 3 degree-3 sumcheck) and print its figures; the cases the ncu "
                         "summaries use.  int_pipes builds bench_int_pipes.cu into build/int_pipes and runs it "
                         "(integer issue rates and field-primitive throughputs)")
    return ap.parse_args()


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def workload_name(a):
    return (f"large-batch commit: {a.rows} rows x 2^{a.log_k} uniform Goldilocks elems, blowup {a.blowup} "
            f"coset NTT to 2^{a.log_k + (a.blowup.bit_length() - 1)} cols, BLAKE3 column hash + Merkle root")


# ----------------------------------------------------------------------------- CPU arm
def cpu_sample(a, rows, steps=1, warmup=0):
    """Times oracle.commit_rows (encode + column hash + Merkle) on `rows` rows of the workload."""
    import numpy as np
    import oracle
    k, n = 1 << a.log_k, (1 << a.log_k) * a.blowup
    cores = os.cpu_count() or 1
    rng = np.random.default_rng(0)
    msg = rng.integers(0, P, size=(rows, k), dtype=np.uint64)
    oracle.lib()
    for _ in range(warmup):
        oracle.commit_rows(msg, n)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.commit_rows(msg, n)
    dt = (time.perf_counter() - t0) / steps
    return {"value": rows * n / dt, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{rows} rows of the workload (encode + column hash + Merkle), C oracle with OpenMP on "
                      f"{cores} threads, {dt:.2f} s per pass"}, dt


def auto_cpu_rows(a):
    """Pick a sample that takes roughly 10-20 s on this host: probe 4 rows, then scale."""
    _, dt = cpu_sample(a, 4)
    rows = int(max(8, min(1024, 15.0 / max(dt / 4, 1e-6))))
    return rows - rows % 4


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = a.cpu_rows or max(8, auto_cpu_rows(a) // max(a.steps + a.warmup, 1))
    base, dt = cpu_sample(a, rows, steps=a.steps, warmup=a.warmup)
    line = {
        "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u64", "data": "synthetic", "impl": "reference",
        "config": {"workload": workload_name(a), "sample_rows_per_step": rows},
        "cpu_baseline": dict(base),
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- GPU arm
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.path = tempfile.NamedTemporaryFile(prefix="clocks_", suffix=".csv", delete=False).name
        self.proc = None
        self.idx = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in open(self.path).read().splitlines():
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def run_native(a):
    import torch
    import torch.distributed as dist

    from verinf_b200 import _lib
    from verinf_b200.commit import RowCommitter

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the native arm has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from verinf_b200.distributed import bind_to_gpu_numa
    numa_bound = bind_to_gpu_numa(local)          # pinned host rows next to the GPU that reads them
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    k, n, rows = 1 << a.log_k, (1 << a.log_k) * a.blowup, a.rows
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    raw = torch.randint(-(1 << 63), (1 << 63) - 1, (rows, k), dtype=torch.int64, device=dev, generator=g)
    msg = raw.view(torch.uint64)
    zero = torch.zeros(1, dtype=torch.uint64, device=dev)
    _lib.check(_lib.LIB.vi_gl_binary_bcast(1, msg.data_ptr(), zero.data_ptr(), 1, msg.data_ptr(), msg.numel(),
                                          _lib.stream_ptr()))          # canonicalise: x >= p -> x - p
    com = RowCommitter(rows, k, k, n, device=dev)
    roots = [torch.empty(32, dtype=torch.uint8, device=dev) for _ in range(world)] if world > 1 else None

    def step():
        root = com.commit(msg)
        if world > 1:
            dist.all_gather(roots, root.contiguous())
        return root

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(a.warmup, 3)):
        step()
    fence()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    _lib.profile_enable(True)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fence()
    ev0.record()
    for _ in range(a.steps):
        root = step()
    ev1.record()
    fence()
    ms = ev0.elapsed_time(ev1)
    prof = _lib.profile_read()
    _lib.profile_enable(False)
    clocks = sampler.stop() if rank == 0 else None
    root_hex = bytes(root.cpu().tolist()).hex()

    # end to end: pinned host input -> H2D -> commit -> D2H root, all inside the timed region
    e2e_ms, host = None, None
    if not a.no_e2e:
        host = torch.empty((rows, k), dtype=torch.uint64).pin_memory()
        host.copy_(msg)
        torch.cuda.synchronize()
        for _ in range(2):
            com.commit_host(host)
        fence()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(a.steps):
            rb = com.commit_host(host)
        t1.record()
        fence()
        e2e_ms = t0.elapsed_time(t1)
        assert rb.hex() == root_hex, "host-path root differs from the device-path root"

    t = torch.tensor([ms, e2e_ms or 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])

    h2d_bytes, d2h_bytes = com.h2d_bytes, com.d2h_bytes
    extra = {}
    if (a.sumcheck or a.extra) and rank == 0:
        extra["sumcheck"] = time_sumcheck(torch, dev)
    if a.extra and rank == 0:
        from verinf_b200 import workloads
        del com, msg, raw, host
        torch.cuda.empty_cache()
        extra["kquant_fused_encode"] = [workloads.kquant_fused_encode(dev, q) for q in ("Q4_K", "Q6_K")]
        extra["layer7b"] = workloads.layer7b_commit_sumcheck(dev)
        extra["field_matmul"] = workloads.field_matmul(dev)
        extra["fold_products"] = workloads.fold_products(dev)

    if rank == 0:
        elems = world * rows * n
        hbm_peak, peak_src = peaks()
        # dominant kernel = the tag with the largest share of device time in the timed region
        total_prof = sum(v[0] for v in prof.values()) or 1.0
        dom = max(prof.items(), key=lambda kv: kv[1][0])
        per_row = {"encode_pass1": 8 * (k + k), "encode_mid": 8 * (k + n), "encode_pass3": 8 * (n + n),
                   "hash_columns": 8 * n}
        # DRAM bytes per message row from ncu captures of these kernels (dram read + write of one launch /
        # rows of that launch), valid for this geometry only; scaled to an average launch
        ncu_per_row = {"encode_pass1": 1.597e6, "encode_mid": 2.515e6, "encode_pass3": 4.343e6,
                       "hash_columns": 2.197e6} if (a.log_k, a.blowup) == (16, 4) else {}
        launches = sum(v[1] for v in prof.values())
        bytes_per_step = rows * per_row.get(dom[0], 0)
        dom_ms_per_step = dom[1][0] / a.steps
        achieved = bytes_per_step / (dom_ms_per_step * 1e-3) / 1e9 if dom_ms_per_step else 0.0
        enc_ms = sum(prof.get(t_, (0, 0))[0] for t_ in ("encode_pass1", "encode_mid", "encode_pass3")) / a.steps
        # integer roofline of the encode: radix-16 butterfly element-stages and full modular multiplies at
        # their ALU-pipe cost measured with the integer-pipe microbenchmark (8.8 and 17.3 ALU lane-ops), against
        # 148 SMs x 64 ALU lanes per clock at the SM clock sampled during the run
        log_n = a.log_k
        stages_per_row = (1 + a.blowup) * k * log_n
        muls_per_row = (1 + a.blowup) * k * 3 + a.blowup * k + k
        alu_ops = rows * (stages_per_row * 8.8 + muls_per_row * 17.3)
        sm_hz = ((clocks or {}).get("sm_mhz") or 1965.0) * 1e6
        alu_floor_ms = alu_ops / (148 * 64 * sm_hz) * 1e3
        line = {
            "metric": METRIC, "value": elems * a.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms / a.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
            "data": "synthetic",
            "config": {"workload": workload_name(a), "rows_per_gpu": rows, "K": k, "N": n,
                       "l2_policy": "inputs (2 GiB) and outputs (8 GiB) exceed L2; no flush needed",
                       "numa_bound": numa_bound,
                       "root": root_hex},
            "roofline": {"bound": "hbm", "kernel": dom[0], "achieved": achieved, "peak": hbm_peak,
                         "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": peak_src,
                         "traffic": (ncu_per_row[dom[0]] * rows * a.steps / dom[1][1]) if dom[0] in ncu_per_row else None,
                         "launches_per_step": dom[1][1] / a.steps,
                         "ms_per_launch": dom[1][0] / dom[1][1],
                         "algorithmic_bytes_per_step": bytes_per_step,
                         "share_of_device_time": dom[1][0] / total_prof},
            "kernels": {t_: {"ms_per_step": v[0] / a.steps, "launches_per_step": v[1] / a.steps,
                             "share": v[0] / total_prof,
                             "gbs": rows * per_row.get(t_, 0) / (v[0] / a.steps * 1e-3) / 1e9 if v[0] else None}
                        for t_, v in prof.items()},
            "encode_only": {"ms_per_step": enc_ms,
                            "gbs_algorithmic": rows * 8 * (k + n) / (enc_ms * 1e-3) / 1e9 if enc_ms else None,
                            "frac_of_hbm": rows * 8 * (k + n) / (enc_ms * 1e-3) / 1e9 / hbm_peak if enc_ms else None},
            "int_roofline": {"bound": "integer ALU pipe (64 lanes/clk/SM)", "encode_floor_ms": alu_floor_ms,
                             "encode_ms": enc_ms, "frac": alu_floor_ms / enc_ms if enc_ms else None},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if e2e_ms:
            line["e2e"] = {"value": elems * a.steps / (e2e_ms * 1e-3), "unit": UNIT,
                           "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                           "ms_per_step": e2e_ms / a.steps}
        if world == 1 and not a.no_cpu:
            crow = a.cpu_rows or auto_cpu_rows(a)
            line["cpu_baseline"], _ = cpu_sample(a, crow)
        line.update(extra)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def time_sumcheck(torch, dev):
    """Degree-3 product of three 2^24 tables, 24 rounds, coins pre-drawn (all rounds + one D2H; the
    claim is the first round's g(0) + g(1))."""
    from verinf_b200 import layergkr_gpu as lg
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    tabs = torch.randint(0, (1 << 62), (3, 1 << 24), dtype=torch.int64, device=dev, generator=g).view(torch.uint64)
    coins = [((i + 1) * 0x9E3779B97F4A7C15) % P for i in range(24)]
    best = None
    for _ in range(3):
        t = tabs.clone()
        prob = lg.SumcheckProblem(t, [(1, [0, 1, 2])])
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ys = prob.run(coins)                       # all rounds queued; g(1) of later rounds derived on the host
        claim = (ys[0][0] + ys[0][1]) % P          # the sum over the hypercube is g_0(0) + g_0(1)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    nbytes = 4 * 3 * (1 << 24) * 8
    return {"ms": best * 1e3, "algorithmic_gbs": nbytes / best / 1e9}


def build_int_pipes():
    """Compiles the integer-pipe / field-primitive microbenchmark (bench_int_pipes.cu) for sm_100a."""
    from verinf_b200.build import _nvcc
    out = ROOT / "build" / "int_pipes"
    src = ROOT / "bench_int_pipes.cu"
    out.parent.mkdir(exist_ok=True)
    if not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
        env = {k_: v for k_, v in os.environ.items() if k_ not in ("CC", "CXX")}
        subprocess.check_call([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
                               "--expt-relaxed-constexpr", "-I", str(ROOT), "-o", str(out), str(src)], env=env)
    return out


def run_micro(a):
    if a.micro == "int_pipes":
        sys.exit(subprocess.call([str(build_int_pipes())]))
    import torch
    from verinf_b200 import workloads
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    if a.micro == "matmul":
        out = workloads.field_matmul(dev, 1024, 2048, 2048)
    elif a.micro == "fold":
        out = workloads.fold_products(dev)
    else:
        out = time_sumcheck(torch, dev)
    print(json.dumps({"micro": a.micro, **out}))


if __name__ == "__main__":
    args = parse()
    if args.micro:
        run_micro(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)
