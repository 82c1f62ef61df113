"""Multi-GPU sharding of the hot path (one process per GPU, torch.distributed).

The reference is single-GPU; this is the sharding the path admits naturally:

* encode: rows are independent -> contiguous row ranges per rank, no communication;
* column hash of ONE tree over all rows: every rank reduces the aligned blocks of its row
  range to non-root BLAKE3 sub-tree chaining values (32 B per column per block), the values
  are all-gathered and every rank folds them into the leaves, then builds the Merkle tree;
* sumcheck: rank g holds the entries i = g (mod G) of every table, so each fold stays local;
  per round the deg+1 partial sums are all-reduced (as 32-bit limbs, summed exactly, then
  reduced mod p); the last log2 G rounds run on the gathered G-entry tables.

The collectives go through torch.distributed (NCCL on GPUs, gloo in the CPU tests); the
local compute is injected (`backend`), so the host logic here is testable without a GPU.
"""
from typing import Callable, List, Sequence, Tuple

import torch
import torch.distributed as dist

P = (1 << 64) - (1 << 32) + 1
CHUNK_ROWS = 128


def split_rows(total_rows: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous [start, end) row ranges, one per rank, cut on 128-row chunk boundaries and as
    even as the chunk count allows (trailing ranks may be empty when there are few chunks)."""
    chunks = max(1, -(-total_rows // CHUNK_ROWS))
    base, extra = divmod(chunks, world)
    out, c = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((min(c * CHUNK_ROWS, total_rows), min((c + n) * CHUNK_ROWS, total_rows)))
        c += n
    return out


def aligned_blocks(start_row: int, end_row: int) -> List[Tuple[int, int, int]]:
    """Greedy decomposition of a chunk-aligned row range into maximal aligned power-of-two chunk
    blocks: [(first_row, n_rows, level)], block = 2^level chunks starting at a multiple of 2^level."""
    if start_row >= end_row:
        return []
    assert start_row % CHUNK_ROWS == 0
    c0, c1 = start_row // CHUNK_ROWS, -(-end_row // CHUNK_ROWS)
    out = []
    while c0 < c1:
        lvl = 0
        while c0 % (2 << lvl) == 0 and c0 + (2 << lvl) <= c1:
            lvl += 1
        r0 = c0 * CHUNK_ROWS
        out.append((r0, min(end_row, (c0 + (1 << lvl)) * CHUNK_ROWS) - r0, lvl))
        c0 += 1 << lvl
    return out


class CudaBackend:
    """Local compute on this rank's GPU through the C ABI."""

    def __init__(self, k_deg, n_lig, master_seed=None):
        from . import cuda_primitives as cp
        self.cp, self.k, self.n, self.seed = cp, k_deg, n_lig, master_seed

    def encode(self, msg, row_offset):
        return self.cp.encode_rows(msg, self.k, self.n, master_seed=self.seed, row_offset=row_offset,
                                   need_polys=False)[1]

    def hash_columns(self, codes):
        return self.cp.hash_columns_streamed(codes)

    def hash_subtree(self, rows, first_chunk, level):
        from ._lib import LIB, check, ptr, scratch, stream_ptr
        n = rows.size(1)
        out = torch.empty((n, 32), dtype=torch.uint8, device=rows.device)
        nb = LIB.vi_hash_subtree_state_bytes(n, level)
        st = scratch(nb, rows.device, "subtree")
        with torch.cuda.device(rows.device):
            check(LIB.vi_hash_subtree(ptr(rows), rows.size(0), n, first_chunk, level, ptr(st), ptr(out), stream_ptr()))
        return out

    def merge(self, cvs, levels):
        import numpy as np
        from ._lib import LIB, check, ptr, stream_ptr
        nb, n, _ = cvs.shape
        lv = np.asarray(levels, dtype=np.int32)
        out = torch.empty((n, 32), dtype=torch.uint8, device=cvs.device)
        with torch.cuda.device(cvs.device):
            check(LIB.vi_hash_merge_subtrees(ptr(cvs), lv.ctypes.data, nb, n, ptr(out), stream_ptr()))
        return out

    def merkle(self, leaves):
        return self.cp.merkle_build_blake3(leaves)


def commit_rows_sharded(msg_local, total_rows: int, backend, group=None, row_offset: int = 0):
    """One commitment over `total_rows` message rows of which this rank holds its split_rows() range.

    Returns (root, levels, codewords_local).  The root equals the single-GPU commit of the
    concatenated rows: encode locally, hash the local aligned blocks to sub-tree chaining values,
    all-gather them (32 bytes per column per block), fold and build the Merkle tree on every rank."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    ranges = split_rows(total_rows, world)
    r0, r1 = ranges[rank]
    assert msg_local.shape[0] == r1 - r0, f"rank {rank} must hold rows [{r0}, {r1})"
    codes = backend.encode(msg_local, row_offset + r0)
    plan = [aligned_blocks(a, b) for a, b in ranges]          # every rank can compute every rank's plan
    n_blocks = sum(len(p) for p in plan)
    if n_blocks < 2:                                          # a single sub-tree would need the root flag inside
        assert world == 1 or all(len(p) == 0 for i, p in enumerate(plan) if i != 0)
        if rank == 0 or world == 1:
            leaves = backend.hash_columns(codes)
        else:
            leaves = torch.empty((codes.shape[1], 32), dtype=torch.uint8, device=codes.device)
        if world > 1:           # src is a global rank: the first member of the group
            dist.broadcast(leaves, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        root, levels = backend.merkle(leaves)
        return root, levels, codes
    mine = [backend.hash_subtree(codes[b0 - r0:b0 - r0 + cnt], b0 // CHUNK_ROWS, lvl) for b0, cnt, lvl in plan[rank]]
    width = max(len(p) for p in plan)
    ncols = codes.shape[1]
    local = torch.zeros((width, ncols, 32), dtype=torch.uint8, device=codes.device)
    for i, cv in enumerate(mine):
        local[i] = cv
    if world > 1:
        gathered = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(gathered, local, group=group)
    else:
        gathered = [local]
    cvs = torch.cat([gathered[r][:len(plan[r])] for r in range(world) if len(plan[r])])
    levels_list = [lvl for p in plan for _, _, lvl in p]
    leaves = backend.merge(cvs.contiguous(), levels_list)
    root, levels = backend.merkle(leaves)
    return root, levels, codes


def _limbs(t_u64: torch.Tensor) -> torch.Tensor:
    """(...,) uint64 -> (..., 2) int64 of 32-bit limbs (lo, hi), on the tensor's device."""
    x = t_u64.contiguous().view(torch.int64)
    return torch.stack([x & 0xFFFFFFFF, (x >> 32) & 0xFFFFFFFF], dim=-1)


def samples_to_host(buf: torch.Tensor, deg: int) -> List[List[int]]:
    """(n_rounds, 8) uint64 samples -> [[g(0..deg)] per round] as Python ints, one copy."""
    import numpy as np
    return buf.view(torch.int64).cpu().numpy().view(np.uint64)[:, :deg + 1].tolist()


def _from_limbs(rows) -> List[int]:
    """[(sum of lo limbs, sum of hi limbs)] -> field elements"""
    return [(int(lo) + (int(hi) << 32)) % P for lo, hi in rows]


def allreduce_field_device(t_u64: torch.Tensor, group=None) -> torch.Tensor:
    """Sum over the ranks of a small tensor of field elements, entirely on the device: returns
    (..., 2) int64 limb sums (exact integers; reduce with _from_limbs after one host copy).
    Collectives have no mod-p sum, so each 64-bit value travels as two 32-bit limbs in int64
    lanes; the integer sum of up to 2^31 ranks cannot overflow."""
    limbs = _limbs(t_u64)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(limbs, op=dist.ReduceOp.SUM, group=group)
    return limbs


def allreduce_field(values: Sequence[int], device, group=None) -> List[int]:
    """Exact sum mod p over the ranks of a few field elements held as Python ints."""
    vals = [int(v) % P for v in values]
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return vals
    limbs = torch.tensor([[v & 0xFFFFFFFF, v >> 32] for v in vals], dtype=torch.int64, device=device)
    dist.all_reduce(limbs, op=dist.ReduceOp.SUM, group=group)
    return _from_limbs(limbs.cpu().tolist())


def shard_table(table: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Entries i = rank (mod world) of a 2^n-entry table: with this split the most-significant-first
    folds of the first n - log2(world) rounds never cross ranks."""
    return table.view(torch.int64)[..., rank::world].contiguous().view(table.dtype)


def _gather_tail(finals_u64: torch.Tensor, world: int, group) -> torch.Tensor:
    """(n_tables,) residual entries of this rank -> (n_tables, world) gathered tables, on the device."""
    mine = finals_u64.contiguous().view(torch.int64)
    if world == 1:
        return mine.reshape(-1, 1).view(torch.uint64)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine, group=group)
    return torch.stack(parts, dim=1).contiguous().view(torch.uint64)


def prove_terms_sharded(local_problem, make_problem: Callable, coin: Callable[[int], int], n_rounds: int,
                        device, group=None, coins: Sequence[int] = None):
    """Sumcheck over tables sharded with shard_table().

    local_problem  this rank's shard (verinf_b200.layergkr_gpu.SumcheckProblem, or any object
                   with round(r or None) -> samples or None and finals() -> [value per table])
    make_problem   builds the same kind of object from an (n_tables, G) uint64 tensor of gathered
                   residual entries, for the last log2(G) rounds
    coins          the challenges when they are known before the sumcheck starts (every call site
                   of the reference pre-draws them, layergkr/full_layer.py:221-224): then nothing is
                   read back per round -- the local rounds are queued, their partial samples are
                   limb-split and all-reduced on the device in one collective, the residual entries
                   all-gathered, the last log2(G) rounds queued, and one host copy ends the proof.
                   Without `coins` the per-round callback `coin(i)` is honoured: one all-reduce
                   (device limbs) and one small host read per round.
    Returns (claim, round_polys, challenges) identical to the unsharded prover's."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    log_g = world.bit_length() - 1
    assert 1 << log_g == world, "world size must be a power of two"
    local_rounds = n_rounds - log_g
    assert local_rounds >= 0, "tables smaller than the world size"
    on_device = hasattr(local_problem, "round_device")
    if coins is not None and on_device:
        return _prove_sharded_queued(local_problem, make_problem, [int(c) % P for c in coins], local_rounds,
                                     n_rounds, world, group)
    from .layergkr_gpu import _interp_at
    polys, chals = [], []
    r, prev = None, None
    for rnd in range(local_rounds):
        if on_device:
            out, skipped = local_problem.round_device(r)
            ys = _from_limbs(allreduce_field_device(out, group).cpu().tolist())     # one host read per round
            if skipped:                                  # g(0) + g(1) = g_prev(r) holds for the global sums
                ys[1] = (_interp_at(prev, r) - ys[0]) % P
        else:
            ys = allreduce_field(local_problem.round(r), device, group)
        polys.append(list(enumerate(ys)))
        prev = ys
        r = (coin(rnd) if coins is None else coins[rnd]) % P
        chals.append(r)
    if local_rounds:
        local_problem.round_device(r) if on_device else local_problem.round(r)   # last local fold
    if log_g:
        if on_device:
            tail = _gather_tail(local_problem.tables[:, 0], world, group)
        else:
            mine = torch.tensor([[v & 0xFFFFFFFF, v >> 32] for v in local_problem.finals()], dtype=torch.int64,
                                device=device)
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine, group=group)
            rows = [[(int(lo) + (int(hi) << 32)) for lo, hi in p.cpu().tolist()] for p in parts]   # [rank][table]
            tail = torch.tensor([[_as_i64(rows[g][t]) for g in range(world)] for t in range(len(rows[0]))],
                                dtype=torch.int64, device=device).view(torch.uint64)
        tail_problem = make_problem(tail)
        r = None
        for rnd in range(local_rounds, n_rounds):
            ys = tail_problem.round(r)
            polys.append(list(enumerate(ys)))
            r = (coin(rnd) if coins is None else coins[rnd]) % P
            chals.append(r)
        tail_problem.round(r)
    claim = (polys[0][0][1] + polys[0][1][1]) % P if polys else \
        allreduce_field([local_problem.claim()], device, group)[0]     # sum over the hypercube = g_0(0) + g_0(1)
    return claim, polys, chals


def _complete_on_device(rows: torch.Tensor, deg: int, coins: Sequence[int]) -> None:
    """g(1) of rows 1.. of an (n, 8) uint64 CUDA sample buffer, in place (vi_sumcheck_complete)."""
    import numpy as np
    from ._lib import LIB, check, ptr, stream_ptr
    if rows.size(0) < 2:
        return
    cs = np.array([int(c) % P for c in coins[:rows.size(0)]], dtype=np.uint64)
    with torch.cuda.device(rows.device):
        check(LIB.vi_sumcheck_complete(ptr(rows), rows.size(0), deg, cs.ctypes.data, stream_ptr()))


def _limbs_to_field_device(limbs: torch.Tensor) -> torch.Tensor:
    """(..., 2) int64 limb sums on a CUDA device -> (...) canonical uint64: lo + hi * 2^32 mod p with the
    library's field kernels (both sums stay below 2^63 < p for up to 2^31 ranks)."""
    from . import cuda_primitives as cp
    lo = limbs[..., 0].contiguous().view(torch.uint64)
    hi = limbs[..., 1].contiguous().view(torch.uint64)
    two32 = torch.full(hi.shape, 1 << 32, dtype=torch.int64, device=hi.device).view(torch.uint64)
    return cp.gl_add(lo, cp.gl_mul(hi, two32))


def _prove_sharded_queued(local_problem, make_problem, coins, local_rounds, n_rounds, world, group):
    """prove_terms_sharded with the challenges known up front; see there."""
    deg = local_problem.deg
    red = None
    if local_rounds:
        buf = local_problem.run_device(coins[:local_rounds])            # (local_rounds, 8), nothing read back
        red = allreduce_field_device(buf[:, :deg + 1], group)           # (local_rounds, deg + 1, 2) limb sums
    tail_buf = None
    if n_rounds > local_rounds:
        tail_problem = make_problem(_gather_tail(local_problem.tables[:, 0], world, group))
        tail_buf = tail_problem.run_device(coins[local_rounds:])
    on_device = (red is None or red.is_cuda) and (tail_buf is None or tail_buf.is_cuda)
    if on_device:
        # recombine the limb sums, fill g(1) of the later rounds and join the two parts on the device: one host copy
        parts = []
        if red is not None:
            rows_dev = torch.zeros((local_rounds, 8), dtype=torch.int64, device=red.device)
            rows_dev[:, :deg + 1] = _limbs_to_field_device(red).view(torch.int64)
            rows_dev = rows_dev.view(torch.uint64)
            _complete_on_device(rows_dev, deg, coins[:local_rounds])
            parts.append(rows_dev)
        if tail_buf is not None:      # the first tail round is evaluated in full; later ones follow from their predecessor
            _complete_on_device(tail_buf, deg, coins[local_rounds:])
            parts.append(tail_buf)
        both = parts[0] if len(parts) == 1 else torch.cat([p.view(torch.int64) for p in parts]).view(torch.uint64)
        out = samples_to_host(both, deg)
    else:
        rows = []
        if red is not None:
            rows += [_from_limbs(r) for r in red.cpu().tolist()]
        n_local = len(rows)
        if tail_buf is not None:
            rows += samples_to_host(tail_buf, deg)
        out = type(local_problem).complete_samples(rows[:n_local], coins[:n_local])
        if tail_buf is not None:
            out += type(local_problem).complete_samples(rows[n_local:], coins[n_local:])
    polys = [list(enumerate(ys)) for ys in out]
    claim = (out[0][0] + out[0][1]) % P
    return claim, polys, list(coins[:n_rounds])


def _as_i64(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def bind_to_gpu_numa(device_index: int) -> bool:
    """Pin this process to the CPUs NVML reports as local to the GPU, so that pinned host buffers
    allocated afterwards (first touch) sit on the GPU's NUMA node.  With one rank per GPU feeding
    gigabytes per step over PCIe this keeps the copies off the inter-socket link.  Only reads
    device properties; returns False (and changes nothing) if anything is unavailable."""
    import os
    try:
        import pynvml
        p = torch.cuda.get_device_properties(device_index)
        pynvml.nvmlInit()
        try:
            bus = f"{p.pci_domain_id:08x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
            h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(p.uuid)).encode())
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        cpus = {64 * w + b for w, m in enumerate(words) for b in range(64) if (int(m) >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if not cpus:
            return False
        os.sched_setaffinity(0, cpus)
        return True
    except Exception:
        return False
