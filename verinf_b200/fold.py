"""Evaluation-domain fold of row products (the q_lin and p_0 transforms of the prover).

Both folds of the reference multiply rows of coefficient polynomials pairwise in the 2K-point
evaluation domain and sum the products over the rows, inverting once at the end:

  * q_lin: `_compute_q_lin_inner_chunk(..., return_eval=True)` (prover/core.py:1892-1911) returns
    sum_i NTT(r_i) * NTT(p_i) for the rows of a chunk;
  * p_0: `compute_p_0_streaming` (prover/core.py:2030-2206) accumulates
    sum_t r_quad[t] * (NTT(px_t) NTT(py_t) + NTT(pa_t) NTT(pz_t)) where px/py/pz are rows selected
    from a cache of encoded rows by index.

The reference composes them from zero-padded copies, two `ntt_forward_batched`, `gl_mul`, a
transposed copy and `gl_matvec`.  Here: one out-of-place zero-extended transform per distinct
row (`ntt_forward_padded`) and one gather-multiply-reduce pass over the transformed rows
(`product_colsum`) that sums the 128-bit products unreduced and reduces once per column.
"""
import torch

from ._lib import LIB, check, ptr, scratch, stream_ptr

_U64 = torch.uint64


def _next_pow2(n):
    p = 1
    while p < n:
        p <<= 1
    return p


def eval_size(k_deg):
    """n_eval of the reference: the smallest power of two >= 2K - 1 (prover/core.py:1900-1903)."""
    return max(2, _next_pow2(2 * k_deg - 1))


def ntt_forward_padded(rows, n_eval):
    """(m, k) coefficient rows -> (m, n_eval) evaluations of the zero-extended rows (same values as
    `pad = zeros(m, n_eval); pad[:, :k] = rows; ntt_forward_batched(pad)`)."""
    if rows.dtype != _U64 or not rows.is_cuda or rows.dim() != 2 or not rows.is_contiguous():
        raise RuntimeError("ntt_forward_padded: expected a contiguous 2-D uint64 CUDA tensor")
    m, k = rows.shape
    out = torch.empty((m, n_eval), dtype=_U64, device=rows.device)
    with torch.cuda.device(rows.device):
        nb = LIB.vi_ntt_scratch_bytes(m, n_eval)
        sc = scratch(nb, rows.device)
        check(LIB.vi_ntt_forward_padded(ptr(rows), m, k, ptr(out), n_eval, ptr(sc), nb, stream_ptr()))
    return out


def product_colsum(EA, EB, weights=None, ia=None, ib=None, out=None):
    """out[j] (+)= sum_i weights[i] * EA[ia[i], j] * EB[ib[i], j].

    EA, EB: (rows, n) uint64 matrices (already in the evaluation domain); ia / ib: optional int64
    CUDA index tensors of equal length T (identity when omitted, then EA and EB must have the same
    number of rows); weights: optional (T,) uint64.  With `out` given the sum is added into it,
    else a new (n,) tensor is returned."""
    for t, name in ((EA, "EA"), (EB, "EB")):
        if t.dtype != _U64 or not t.is_cuda or t.dim() != 2 or not t.is_contiguous():
            raise RuntimeError(f"product_colsum: {name} must be a contiguous 2-D uint64 CUDA tensor")
    n = EA.size(1)
    if EB.size(1) != n:
        raise RuntimeError("product_colsum: column counts differ")
    if (ia is None) != (ib is None):
        raise RuntimeError("product_colsum: give both index tensors or neither")
    if ia is None:
        if EA.size(0) != EB.size(0):
            raise RuntimeError("product_colsum: row counts differ")
        T = EA.size(0)
    else:
        for t, lim in ((ia, EA.size(0)), (ib, EB.size(0))):
            if t.dtype != torch.int64 or not t.is_cuda or t.dim() != 1 or not t.is_contiguous():
                raise RuntimeError("product_colsum: indices must be contiguous 1-D int64 CUDA tensors")
            if t.numel() and (int(t.min()) < 0 or int(t.max()) >= lim):
                raise RuntimeError("product_colsum: row index out of range")
        T = ia.numel()
        if ib.numel() != T:
            raise RuntimeError("product_colsum: index lengths differ")
    if weights is not None:
        if weights.dtype != _U64 or not weights.is_cuda or weights.numel() != T or not weights.is_contiguous():
            raise RuntimeError("product_colsum: weights must be a contiguous uint64 CUDA tensor with one entry per row")
    accumulate = out is not None
    if out is None:
        out = torch.empty(n, dtype=_U64, device=EA.device)
    elif out.dtype != _U64 or out.numel() != n or not out.is_contiguous():
        raise RuntimeError("product_colsum: bad output tensor")
    with torch.cuda.device(EA.device):
        nb = LIB.vi_product_colsum_scratch_bytes(T, n)
        sc = scratch(nb, EA.device)
        check(LIB.vi_product_colsum(ptr(EA), ptr(EB), n, ptr(ia), ptr(ib), ptr(weights), T, ptr(out),
                                    1 if accumulate else 0, ptr(sc), nb, stream_ptr()))
    return out


def fold_products_eval(A, B, weights=None, out=None):
    """sum_i weights[i] * NTT(A_i) * NTT(B_i) in the n_eval-point domain for (m, K) coefficient rows:
    the value `_compute_q_lin_inner_chunk(return_eval=True)` returns for r_i = A_i, p_i = B_i
    (prover/core.py:1892-1911), and one chunk's `weighted_eval` of compute_p_0_streaming with
    weights = r_quad (prover/core.py:2166-2181).  `ntt_inverse` of the accumulated result, cut to
    2K - 1 coefficients, is the folded polynomial."""
    if A.shape != B.shape:
        raise RuntimeError("fold_products_eval: shapes differ")
    n_eval = eval_size(A.size(1))
    return product_colsum(ntt_forward_padded(A, n_eval), ntt_forward_padded(B, n_eval), weights, out=out)
