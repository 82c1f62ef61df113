"""CPU, world_size 2 and 4 over gloo: the host-side sharding logic of verinf_b200.distributed
(row split, aligned-block plan, chaining-value gather and fold, limb-split field all-reduce,
sharded sumcheck) with the CPU oracle standing in for the per-rank GPU kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from verinf_b200 import distributed as D

P = oracle.P


def _u64(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int64)).view(torch.uint64)


def _np(t):
    return t.contiguous().view(torch.int64).numpy().view(np.uint64)


class OracleBackend:
    """Per-rank compute of commit_rows_sharded on CPU tensors through the oracle."""

    def __init__(self, k, n):
        self.k, self.n = k, n

    def encode(self, msg, row_offset):
        m = _np(msg)
        padded = np.zeros((m.shape[0], self.k), dtype=np.uint64)
        padded[:, :m.shape[1]] = m
        if m.shape[0] == 0:
            return _u64(np.zeros((0, self.n), dtype=np.uint64))
        return _u64(oracle.encode_rows(padded, self.n, want_polys=False)[1])

    def hash_columns(self, codes):
        return torch.from_numpy(oracle.hash_columns(_np(codes)))

    def hash_subtree(self, rows, first_chunk, level):
        return torch.from_numpy(oracle.hash_subtree(_np(rows), first_chunk))

    def merge(self, cvs, levels):
        return torch.from_numpy(oracle.hash_merge_subtrees(cvs.numpy(), levels))

    def merkle(self, leaves):
        lv = oracle.merkle_levels(leaves.numpy())
        return torch.from_numpy(lv[-1].reshape(-1).copy()), [torch.from_numpy(x.copy()) for x in lv]


class PySumcheck:
    """Reference-shaped local sumcheck problem on Python ints (layergkr/sumcheck.py:153-226 loop)."""

    def __init__(self, tables, terms):
        self.t = [[int(v) for v in row] for row in tables]
        self.terms = terms
        self.deg = max(len(f) for _, f in terms)

    def claim(self):
        acc = 0
        for i in range(len(self.t[0])):
            for c, fs in self.terms:
                p = c
                for k in fs:
                    p = p * self.t[k][i] % P
                acc += p
        return acc % P

    def round(self, r):
        if r is not None:
            h = len(self.t[0]) // 2
            self.t = [[(f[i] + r * (f[h + i] - f[i])) % P for i in range(h)] for f in self.t]
        if len(self.t[0]) < 2:
            return None
        h = len(self.t[0]) // 2
        out = []
        for x in range(self.deg + 1):
            acc = 0
            for i in range(h):
                for c, fs in self.terms:
                    p = c
                    for k in fs:
                        f = self.t[k]
                        p = p * ((f[i] + x * (f[h + i] - f[i])) % P) % P
                    acc += p
            out.append(acc % P)
        return out

    def finals(self):
        return [f[0] for f in self.t]


class TensorSumcheck(PySumcheck):
    """PySumcheck behind the device-resident interface of layergkr_gpu.SumcheckProblem
    (round_device / run_device / tables / complete_samples) on CPU tensors, including its
    convention that g(1) is left 0 after the first round."""

    def __init__(self, tables, terms):
        super().__init__(tables, terms)
        self._seen = False

    @property
    def tables(self):
        return _u64(np.array(self.t, dtype=np.uint64))

    def round_device(self, r):
        ys = self.round(r)
        if ys is None:
            return None, False
        skip = r is not None and self._seen
        self._seen = True
        if skip:
            ys[1] = 0
        return _u64(np.array(ys, dtype=np.uint64)), skip

    def run_device(self, coins):
        buf = np.zeros((len(coins), 8), dtype=np.uint64)
        r = None
        for i, c in enumerate(coins):
            ys = self.round(r)
            if i:
                ys[1] = 0
            buf[i, :len(ys)] = ys
            r = c
        if coins:
            self.round(r)
        return _u64(buf)

    @staticmethod
    def complete_samples(rows, coins, prev=None, prev_coin=None):
        from verinf_b200.layergkr_gpu import SumcheckProblem
        return SumcheckProblem.complete_samples(rows, coins, prev, prev_coin)


def _worker(rank, world, port, total_rows, ell, k, n, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(99)
        msg = rng.integers(0, P, size=(total_rows, ell), dtype=np.uint64)
        r0, r1 = D.split_rows(total_rows, world)[rank]
        root, levels, codes = D.commit_rows_sharded(_u64(msg[r0:r1]), total_rows, OracleBackend(k, n))
        # field all-reduce
        vals = [(rank + 1) * (P - 1) % P, P - 1, 5 + rank]
        red = D.allreduce_field(vals, "cpu")
        # sharded sumcheck, 2^6 entries, degree 3 product + a second term
        tabs = rng.integers(0, P, size=(3, 64), dtype=np.uint64)
        terms = [(1, [0, 1, 2]), (P - 2, [1, 0])]
        coins = [int(c) for c in rng.integers(0, P, size=6, dtype=np.uint64)]
        local = PySumcheck([row[rank::world] for row in tabs.tolist()], terms)
        claim, polys, chals = D.prove_terms_sharded(
            local, lambda t: PySumcheck(_np(t).tolist(), terms), lambda i: coins[i], 6, "cpu")
        # the same proof through the device-resident interface: per-round callback, then queued coins
        for kw in ({}, {"coins": coins}):
            loc = TensorSumcheck([row[rank::world] for row in tabs.tolist()], terms)
            c2, p2, ch2 = D.prove_terms_sharded(loc, lambda t: TensorSumcheck(_np(t).tolist(), terms),
                                                lambda i: coins[i], 6, "cpu", **kw)
            assert (c2, p2, ch2) == (claim, polys, chals), f"device-interface path {kw and 'queued'} differs"
        q.put((rank, bytes(root.tolist()), red, claim, [[y for _, y in rp] for rp in polys], chals))
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world,total_rows", [(2, 700), (4, 1000), (2, 100)])
def test_sharded_commit_and_sumcheck_match_single_process(world, total_rows):
    ell, k, n = 24, 32, 128
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, total_rows, ell, k, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    rng = np.random.default_rng(99)
    msg = rng.integers(0, P, size=(total_rows, ell), dtype=np.uint64)
    padded = np.zeros((total_rows, k), dtype=np.uint64)
    padded[:, :ell] = msg
    want_root = oracle.commit_rows(padded, n)
    tabs = rng.integers(0, P, size=(3, 64), dtype=np.uint64)
    terms = [(1, [0, 1, 2]), (P - 2, [1, 0])]
    coins = [int(c) for c in rng.integers(0, P, size=6, dtype=np.uint64)]
    claim, samples, _ = oracle.sumcheck(tabs, terms, coins)
    want_red = [sum((r + 1) * (P - 1) % P for r in range(world)) % P, world * (P - 1) % P,
                sum(5 + r for r in range(world)) % P]
    for rank, root, red, c, polys, chals in results:
        assert root == want_root, f"rank {rank}: sharded root differs"
        assert red == want_red
        assert c == claim and chals == coins
        assert polys == [[int(v) for v in row] for row in samples]


def test_split_and_blocks():
    assert D.split_rows(4096, 8) == [(i * 512, (i + 1) * 512) for i in range(8)]
    assert D.split_rows(100, 2) == [(0, 100), (100, 100)]
    assert D.split_rows(1000, 3) == [(0, 384), (384, 768), (768, 1000)]
    assert D.aligned_blocks(512, 1024) == [(512, 512, 2)]
    assert D.aligned_blocks(128, 1000) == [(128, 128, 0), (256, 256, 1), (512, 488, 2)]
    assert D.aligned_blocks(384, 768) == [(384, 128, 0), (512, 256, 1)]
    assert D.aligned_blocks(100, 100) == []
    for total in (1, 128, 129, 1000, 4096, 5000):
        for world in (1, 2, 3, 8):
            rs = D.split_rows(total, world)
            assert rs[0][0] == 0 and rs[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(rs, rs[1:]))
            covered = [blk for a, b in rs for blk in D.aligned_blocks(a, b)]
            assert sum(c for _, c, _ in covered) == total
            for r0, cnt, lvl in covered:
                assert (r0 // 128) % (1 << lvl) == 0 and -(-cnt // 128) == 1 << lvl
