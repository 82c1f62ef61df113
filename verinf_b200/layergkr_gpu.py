"""Device-resident versions of the layergkr/gpu.py entry points (same names, argument meaning
and return values): `encode_batch_ntt`, `hash_and_tree`, `prove_terms_gpu` on the hot path
(layergkr/gpu.py:141-203, 274-289, 350-410) and the helpers around them (`encode_batch`,
`encode_batch_t`, `linear_combination`, `combine_t`, `column`, `levels_to_host`, `gl_sum`,
`fold_t`, layergkr/gpu.py:92-126, 256-347), so the module can stand in for layergkr.gpu.

`prove_terms_gpu` keeps the reference's per-round `coin` callback, but each round is one
fused fold+evaluate launch and one small D2H copy of the deg+1 samples, instead of ~10
elementwise launches and a host sync per sample point.
"""
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from . import cuda_primitives as cp
from ._lib import LIB, check, ptr, scratch, stream_ptr

P = cp.P
_MAX_FAC = 4


def encode_batch_ntt(cfg, messages):
    """messages: (rows, <=K_DEG) device tensor or Python rows of <= ELL values -> (rows, N_LIG)
    codewords on the coset 7*<w_N>; unused slots up to K_DEG are zero (layergkr convention)."""
    if not hasattr(messages, "shape"):
        src = [list(m) + [0] * (cfg.ELL - len(m)) for m in messages]
        messages = torch.tensor(src, dtype=torch.uint64, device="cuda")
    _, codes = cp.encode_rows(messages.contiguous(), cfg.K_DEG, cfg.N_LIG, need_polys=False)
    return codes


def hash_and_tree(cfg, mat):
    """Column digests + Merkle tree on the device; returns (root bytes, levels tensors)."""
    dig = cp.hash_columns_streamed(mat.contiguous())
    root_t, levels_t = cp.merkle_build_blake3(dig)
    return bytes(root_t.cpu().tolist()), levels_t


def available() -> bool:
    """True when the CUDA library is loaded and a device is present (layergkr/gpu.py:76-77)."""
    return torch.cuda.is_available()


def _messages_tensor(cfg, messages):
    if hasattr(messages, "shape"):
        return messages.contiguous()
    src = [[int(v) % P for v in m] + [0] * (cfg.ELL - len(m)) for m in messages]
    return torch.tensor(src, dtype=torch.uint64, device="cuda")


def encode_batch_t(cfg, messages):
    """Encode to a device tensor (layergkr/gpu.py:256-271).  The reference multiplies by the
    ELL x N Lagrange matrix; the NTT route gives the same codewords (the equivalence the
    reference pins in selftest_ntt, layergkr/gpu.py:206-253) without building that matrix."""
    return encode_batch_ntt(cfg, _messages_tensor(cfg, messages))


def encode_batch(cfg, messages) -> List[List[int]]:
    """Encode and return Python rows (layergkr/gpu.py:92-110)."""
    codes = encode_batch_t(cfg, messages)
    return [[int(v) for v in row] for row in codes.view(torch.int64).cpu().numpy().view(np.uint64).tolist()]


def combine_t(cfg, mat, coeffs: Sequence[int]):
    """sum_i coeffs[i] * mat[i] as a (1, N) device tensor (layergkr/gpu.py:301-308); the matrix is
    streamed once by the thin-product kernel."""
    A = torch.tensor([[int(c) % P for c in coeffs]], dtype=torch.uint64, device=mat.device)
    return cp.gl_matmul(A, mat.contiguous())


def linear_combination(cfg, codewords, coeffs: Sequence[int]) -> List[int]:
    """sum_i coeffs[i] * codewords[i] for Python rows (layergkr/gpu.py:113-123)."""
    B = torch.tensor([[int(v) % P for v in c] for c in codewords], dtype=torch.uint64, device="cuda")
    out = combine_t(cfg, B, coeffs)[0]
    return [int(v) for v in out.view(torch.int64).cpu().numpy().view(np.uint64).tolist()]


def column(mat, col: int) -> List[int]:
    """One codeword column on the host (layergkr/gpu.py:311-316)."""
    from .commit import open_columns
    out = open_columns(mat.contiguous(), [int(col)])[0]
    return [int(v) for v in out.view(torch.int64).cpu().numpy().view(np.uint64).tolist()]


def levels_to_host(levels_t) -> List[List[bytes]]:
    """The whole tree as host byte strings (layergkr/gpu.py:292-298).  For the T opening paths
    alone `commit.merkle_paths` moves T*depth*33 bytes instead."""
    out = []
    for lvl in levels_t:
        arr = lvl.cpu().numpy()
        out.append([arr[r].tobytes() for r in range(arr.shape[0])])
    return out


def gl_sum(t):
    """Field sum of a device vector as a 1-element tensor (layergkr/gpu.py:326-338): one thin
    product with a row of ones per 1024 columns, then the 1024 partial sums the same way."""
    v = t.reshape(-1).contiguous()
    while v.numel() > 1:
        n = v.numel()
        cols = 1024 if n > 1024 else 1
        rows = -(-n // cols)
        if rows * cols != n:
            pad = torch.zeros(rows * cols, dtype=torch.int64, device=v.device)
            pad[:n] = v.view(torch.int64)
            v = pad.view(torch.uint64)
        ones = torch.ones((1, rows), dtype=torch.int64, device=v.device).view(torch.uint64)
        v = cp.gl_matmul(ones, v.view(torch.int64).view(rows, cols).view(torch.uint64)).reshape(-1)
    return v


def fold_t(f, r_t):
    """(f[:h] + r*(f[h:] - f[:h])) mod p on the device (layergkr/gpu.py:341-347); r_t is a
    1-element tensor."""
    h = f.numel() // 2
    lo, hi = f[:h].contiguous(), f[h:2 * h].contiguous()
    return cp.gl_add(lo, cp.gl_mul_rowvec(cp.gl_sub(hi, lo).reshape(h, 1), r_t.reshape(1)).reshape(h))


class SumcheckProblem:
    """Tables and term structure of a sum-of-products sumcheck, resident on the device."""

    def __init__(self, tables: torch.Tensor, terms: Sequence):
        """tables: (n_tables, size) uint64 CUDA tensor (folded in place by `round`);
        terms: [(coef, [table indices])]."""
        assert tables.dtype == torch.uint64 and tables.is_cuda and tables.dim() == 2 and tables.is_contiguous()
        self.tables = tables
        self.size = tables.size(1)
        self.n_tables = tables.size(0)
        self.deg = max(len(f) for _, f in terms)
        self._coefs = np.array([c % P for c, _ in terms], dtype=np.uint64)
        self._nfac = np.array([len(f) for _, f in terms], dtype=np.int32)
        fac = np.zeros((len(terms), _MAX_FAC), dtype=np.int32)
        for t, (_, f) in enumerate(terms):
            if len(f) > _MAX_FAC:
                raise RuntimeError(f"sumcheck: at most {_MAX_FAC} factors per term")
            fac[t, :len(f)] = f
        self._fac = fac
        self.n_terms = len(terms)
        dev = tables.device
        self._out = torch.empty(8, dtype=torch.uint64, device=dev)
        self._partials = scratch(LIB.vi_sumcheck_scratch_bytes(), dev, "sumcheck")
        self._host = torch.empty(8, dtype=torch.uint64).pin_memory()
        self._prev = None       # samples of the previous round (to derive g(1) of the next one)
        self._seen_round = False

    def _args(self):
        return (self.tables.size(1), self.n_tables, self.size, self.n_terms,
                self._coefs.ctypes.data, self._nfac.ctypes.data, self._fac.ctypes.data)

    def _read(self, n) -> List[int]:
        self._host.copy_(self._out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return [int(v) for v in self._host[:n].tolist()]

    def claim(self) -> int:
        with torch.cuda.device(self.tables.device):
            check(LIB.vi_sumcheck_claim(ptr(self.tables), *self._args(), ptr(self._out), ptr(self._partials),
                                        stream_ptr()))
        return self._read(1)[0]

    def round_device(self, r: Optional[int]):
        """Fold with r (None on the first round) and launch the evaluation of the next round without
        reading anything back.  Returns (samples, skipped): `samples` is a device view of g(0..deg)
        (valid until the next launch on this problem), or None once the tables are down to one entry;
        with `skipped` True g(1) was not computed (written as 0) and follows from
        g(0) + g(1) = g_prev(r).  For callers that combine the samples of several shards on the
        device before any host read."""
        fold = r is not None
        skip = fold and self._seen_round
        with torch.cuda.device(self.tables.device):
            check(LIB.vi_sumcheck_round(ptr(self.tables), *self._args(), int(fold) | (2 if skip else 0),
                                        (r or 0) % P, ptr(self._out), ptr(self._partials), stream_ptr()))
        if fold:
            self.size //= 2
        if self.size < 2:
            return None, False
        self._seen_round = True
        return self._out[:self.deg + 1], skip

    def round(self, r: Optional[int]) -> Optional[List[int]]:
        """Fold with r (None on the first round), then return the samples g(0..deg) of the
        current tables, or None once the tables are down to a single entry."""
        # after the first round g(1) is not computed on the device: g(0) + g(1) = g_prev(r)
        out, skip = self.round_device(r)
        if out is None:
            return None
        ys = self._read(self.deg + 1)
        if skip:
            ys[1] = (_interp_at(self._prev, r % P) - ys[0]) % P
        self._prev = ys
        return ys

    def run_device(self, coins: Sequence[int]):
        """All rounds queued back to back for challenges known up front; nothing is read back.
        Returns the (n_rounds, 8) uint64 device buffer of samples: row i holds g_i(0..deg) with
        g_i(1) left 0 for i >= 1 (see complete_samples)."""
        n_rounds = self.size.bit_length() - 1
        assert len(coins) == n_rounds
        buf = torch.zeros((max(n_rounds, 1), 8), dtype=torch.uint64, device=self.tables.device)
        if n_rounds:
            cs = np.array([int(c) % P for c in coins], dtype=np.uint64)
            with torch.cuda.device(self.tables.device):
                check(LIB.vi_sumcheck_run(ptr(self.tables), *self._args(), cs.ctypes.data, n_rounds, ptr(buf),
                                          ptr(self._partials), stream_ptr()))
        self.size = 1
        return buf[:n_rounds]

    @staticmethod
    def complete_samples(rows: List[List[int]], coins: Sequence[int], prev: Optional[List[int]] = None,
                         prev_coin: Optional[int] = None) -> List[List[int]]:
        """Fills the g(1) that the queued rounds leave out: g_i(1) = g_{i-1}(coins[i-1]) - g_i(0).
        Row 0 is complete unless `prev` (the samples of the round before it) is given."""
        out = [list(r) for r in rows]
        for i in range(len(out)):
            if i == 0 and prev is None:
                continue
            p_ys, p_r = (prev, prev_coin) if i == 0 else (out[i - 1], coins[i - 1])
            out[i][1] = (_interp_at(p_ys, int(p_r) % P) - out[i][0]) % P
        return out

    def run(self, coins: Sequence[int]):
        """All rounds back to back for challenges known up front (every call site of the reference
        pre-draws its coins from the transcript before the sumcheck starts): no host round trip per
        round, one D2H copy of all samples at the end.  Returns [[g(0..deg)] per round]."""
        n_rounds = len(coins)
        buf = self.run_device(coins)
        if n_rounds > 1:        # g(1) of the later rounds on the device too: the host only converts
            cs = np.array([int(c) % P for c in coins], dtype=np.uint64)
            with torch.cuda.device(self.tables.device):
                check(LIB.vi_sumcheck_complete(ptr(buf), n_rounds, self.deg, cs.ctypes.data, stream_ptr()))
        out = samples_to_host(buf, self.deg)
        self._prev = out[-1] if out else None
        return out

    def finals(self) -> List[int]:
        return [int(v) for v in self.tables[:, 0].cpu().tolist()]


_MAX_TABLES, _MAX_TERMS = 8, 8          # per launch of the sumcheck kernels (csrc/sumcheck.cu)


class TermGroups:
    """A sum of products with more tables or terms than one kernel launch takes (a layer's gate batch,
    layergkr/relations.py:103-124, has hundreds): the sum is linear in its terms, so the terms are split
    into groups that fit, every group is its own SumcheckProblem folded with the same challenges, and the
    round samples are added.  A group of lower degree is extended to the common number of samples by
    evaluating its round polynomial at the further nodes.  Same interface as SumcheckProblem."""

    def __init__(self, rows: Sequence[torch.Tensor], plan: Sequence):
        self.deg = max(len(idx) for _, idx in plan)
        groups, cur, used = [], [], set()
        for c, idx in plan:
            if cur and (len(cur) == _MAX_TERMS or len(used | set(idx)) > _MAX_TABLES):
                groups.append(cur)
                cur, used = [], set()
            cur.append((c, idx))
            used |= set(idx)
        groups.append(cur)
        self.problems = []
        for g in groups:
            need = sorted({i for _, idx in g for i in idx})
            at = {t: j for j, t in enumerate(need)}
            tables = torch.stack([rows[t].view(torch.int64) for t in need]).view(torch.uint64).contiguous()
            self.problems.append(SumcheckProblem(tables, [(c, [at[i] for i in idx]) for c, idx in g]))
        self.size = self.problems[0].size

    def _add(self, per_group: Sequence[List[int]]) -> List[int]:
        n = self.deg + 1
        out = [0] * n
        for ys in per_group:
            ys = list(ys) + [_interp_at(ys, x) for x in range(len(ys), n)]
            out = [(a + b) % P for a, b in zip(out, ys)]
        return out

    def claim(self) -> int:
        return sum(p.claim() for p in self.problems) % P

    def round(self, r: Optional[int]) -> Optional[List[int]]:
        res = [p.round(r) for p in self.problems]
        self.size = self.problems[0].size
        return None if res[0] is None else self._add(res)

    def run(self, coins: Sequence[int]) -> List[List[int]]:
        per = [p.run(coins) for p in self.problems]
        self.size = 1
        return [self._add([g[i] for g in per]) for i in range(len(coins))]


def samples_to_host(buf: torch.Tensor, deg: int) -> List[List[int]]:
    """(n_rounds, 8) uint64 device samples -> [[g(0..deg)] per round] as Python ints, one copy."""
    host = buf.view(torch.int64).cpu().numpy().view(np.uint64)
    return host[:, :deg + 1].tolist()


_INV_DEN = {}     # n -> [1 / prod_{j != i} (i - j) mod p for i < n]  (Lagrange weights of the nodes 0..n-1)


def _interp_at(ys: Sequence[int], r: int) -> int:
    """Value at r of the polynomial of degree < len(ys) through (0, ys[0]), (1, ys[1]), ..."""
    n = len(ys)
    if r < n:
        return ys[r]
    inv = _INV_DEN.get(n)
    if inv is None:
        inv = []
        for i in range(n):
            den = 1
            for j in range(n):
                if j != i:
                    den = den * ((i - j) % P) % P
            inv.append(pow(den, P - 2, P))
        _INV_DEN[n] = inv
    diffs = [(r - j) % P for j in range(n)]
    total = 0
    for i, y in enumerate(ys):
        num = 1
        for j in range(n):
            if j != i:
                num = num * diffs[j] % P
        total = (total + y * num % P * inv[i]) % P
    return total


def _poly_eval(coeffs, x, p):
    acc = 0
    for c in reversed(coeffs):
        acc = (acc * x + c) % p
    return acc


def prove_terms_gpu(terms, coin: Callable[[int], int], field_p: int = P, mask=None, mu0: int = 0,
                    coins: Optional[Sequence[int]] = None, predraw: bool = False):
    """Sumcheck prover for sum_x sum_k c_k prod_j f_kj(x): returns
    (claim, round_polys [[(x, y), ...] per round], challenges, final_mask).

    `terms` is [(coef, [factor, ...])] where a factor is a Python sequence or a 1-D uint64
    CUDA tensor; factors that are the same object share one device table.  When the challenges are
    known up front pass them as `coins` (then `coin` is not called): all rounds are queued without a
    host round trip.  `predraw=True` does the same by calling coin(0), ..., coin(n_rounds - 1) before
    the first round; valid when `coin` depends on the round index alone, which the reference's
    interface implies (the callback receives nothing else, layergkr/gpu.py:402) and its call sites do
    (layergkr/relations.py:122-123 draws all challenges from the transcript, then passes
    `lambda i: coins[i]`).  The mask of a zero-knowledge proof only touches the scalar samples
    (layergkr/gpu.py:392-396), so masked proofs are queued too."""
    assert field_p == P
    uniq, index, plan = [], {}, []
    for c, fs in terms:
        idx = []
        for f in fs:
            key = id(f)
            if key not in index:
                index[key] = len(uniq)
                uniq.append(f)
            idx.append(index[key])
        plan.append((c % P, idx))
    rows = []
    for f in uniq:
        if isinstance(f, torch.Tensor):
            rows.append(f.to(device="cuda").reshape(-1))
        else:
            rows.append(torch.tensor([int(x) % P for x in f], dtype=torch.uint64, device="cuda"))
    if len(rows) > _MAX_TABLES or len(plan) > _MAX_TERMS:
        prob = TermGroups(rows, plan)
    else:
        tables = torch.stack([r.view(torch.int64) for r in rows]).view(torch.uint64).contiguous()
        prob = SumcheckProblem(tables, plan)
    n_rounds = prob.size.bit_length() - 1
    deg = prob.deg
    mu = mu0 % P
    round_polys, challenges = [], []
    if coins is None and predraw:
        coins = [coin(rnd) for rnd in range(n_rounds)]
    if coins is not None and n_rounds > 0:
        challenges = [int(c) % P for c in coins]
        all_ys = prob.run(challenges)
        claim = (all_ys[0][0] + all_ys[0][1] + mu) % P       # the sum over the hypercube is g_0(0) + g_0(1)
        for ys, r in zip(all_ys, challenges):
            samples = list(enumerate(ys))
            if mask is not None:
                h = mask(deg, mu)
                samples = [(x, (y + _poly_eval(h, x, P)) % P) for x, y in samples]
                mu = _poly_eval(h, r, P)
            round_polys.append(samples)
        return claim, round_polys, challenges, mu
    claim = (prob.claim() + mu) % P
    r = None
    for rnd in range(n_rounds):
        ys = prob.round(r)
        samples = list(enumerate(ys))
        if mask is not None:
            h = mask(deg, mu)
            samples = [(x, (y + _poly_eval(h, x, P)) % P) for x, y in samples]
        round_polys.append(samples)
        r = coin(rnd) % P
        challenges.append(r)
        if mask is not None:
            mu = _poly_eval(h, r, P)
    if n_rounds:
        prob.round(r)          # last fold: tables collapse to their evaluation at the challenge point
    return claim, round_polys, challenges, mu
