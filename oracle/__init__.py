"""ctypes front end of the CPU oracle (oracle/verinf_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by the
benchmark's CPU-baseline leg.  The shipped CUDA path never imports this.
"""
import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "libverinf_oracle.so"
P = (1 << 64) - (1 << 32) + 1
_lib = None


def build(force: bool = False) -> Path:
    src = _HERE / "verinf_oracle.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.check_call(["make", "-C", str(_HERE), "-B", "libverinf_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_SO))
        u64, i64, p = C.c_uint64, C.c_int64, C.c_void_p
        for name in ("or_gl_add", "or_gl_sub", "or_gl_mul", "or_gl_pow"):
            getattr(L, name).restype = u64
            getattr(L, name).argtypes = [u64, u64]
        L.or_gl_inv.restype = u64; L.or_gl_inv.argtypes = [u64]
        L.or_root_of_unity.restype = u64; L.or_root_of_unity.argtypes = [u64]
        L.or_fold_products_eval.argtypes = [p, i64, p, i64, i64, p, p, p, i64, i64, p]
        L.or_fold_products_eval.restype = None
        L.or_gl_matmul.argtypes = [p, p, p, i64, i64, i64]; L.or_gl_matmul.restype = None
        L.or_ntt.argtypes = [p, i64, C.c_int]; L.or_ntt.restype = None
        L.or_ntt_batched.argtypes = [p, i64, i64, C.c_int]; L.or_ntt_batched.restype = None
        L.or_encode_rows.argtypes = [p, i64, i64, i64, p, p]; L.or_encode_rows.restype = None
        L.or_blake3.argtypes = [p, i64, p]; L.or_blake3.restype = None
        L.or_hash_columns.argtypes = [p, i64, i64, p]; L.or_hash_columns.restype = None
        L.or_merkle_total_nodes.argtypes = [i64]; L.or_merkle_total_nodes.restype = i64
        L.or_merkle_levels.argtypes = [p, i64, p]; L.or_merkle_levels.restype = C.c_int
        L.or_row_prg.argtypes = [p, i64, i64, i64, p]; L.or_row_prg.restype = None
        L.or_row_prg_indexed.argtypes = [p, p, i64, i64, p]; L.or_row_prg_indexed.restype = None
        L.or_challenge.argtypes = [p, p, C.c_int, u64]; L.or_challenge.restype = u64
        L.or_kquant_to_field.argtypes = [p, i64, C.c_int, C.c_double, p]
        L.or_kquant_to_field.restype = C.c_int
        L.or_signed_to_field.argtypes = [p, i64, p]; L.or_signed_to_field.restype = None
        L.or_sumcheck.argtypes = [p, C.c_int, i64, C.c_int, p, p, p, C.c_int, p, p, p, p]
        L.or_sumcheck.restype = C.c_int
        L.or_commit_rows.argtypes = [p, i64, i64, i64, p]; L.or_commit_rows.restype = None
        L.or_hash_subtree.argtypes = [p, i64, i64, i64, p]; L.or_hash_subtree.restype = None
        L.or_hash_merge_subtrees.argtypes = [p, p, C.c_int, i64, p]; L.or_hash_merge_subtrees.restype = C.c_int
        L.or_set_threads.argtypes = [C.c_int]; L.or_set_threads.restype = C.c_int
        _lib = L
    return _lib


def set_threads(n: int = 0) -> int:
    """Sets the OpenMP thread count of the oracle's loops (n > 0) and returns the count in effect.
    A launcher's OMP_NUM_THREADS (torchrun exports 1) is overridden, not inherited."""
    if n > 0:
        os.environ["OMP_NUM_THREADS"] = str(n)
    return int(lib().or_set_threads(int(n)))


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def _u64(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint64))


# ---- field -------------------------------------------------------------
def gl_add(a, b): return lib().or_gl_add(int(a), int(b))
def gl_sub(a, b): return lib().or_gl_sub(int(a), int(b))
def gl_mul(a, b): return lib().or_gl_mul(int(a), int(b))
def gl_pow(a, e): return lib().or_gl_pow(int(a), int(e))
def gl_inv(a): return lib().or_gl_inv(int(a))
def root_of_unity(n): return lib().or_root_of_unity(int(n))


def gl_matmul(A, B):
    A, B = _u64(A), _u64(B)
    m, k = A.shape
    k2, n = B.shape
    assert k == k2
    out = np.empty((m, n), dtype=np.uint64)
    lib().or_gl_matmul(_ptr(A), _ptr(B), _ptr(out), m, k, n)
    return out


# ---- NTT / encode ------------------------------------------------------
def ntt(a, invert=False):
    """Natural-order length-n transform of a 1-D uint64 array (returns a copy)."""
    a = _u64(a).copy()
    lib().or_ntt(_ptr(a), a.size, int(bool(invert)))
    return a


def ntt_batched(rows, invert=False):
    rows = _u64(rows).copy()
    m, n = rows.shape
    lib().or_ntt_batched(_ptr(rows), m, n, int(bool(invert)))
    return rows


def encode_rows(padded, n_lig, want_polys=True, want_codes=True):
    """padded: (m, K) values at the K-th roots of unity -> (polys (m,K), codes (m,N))."""
    padded = _u64(padded)
    m, k = padded.shape
    polys = np.empty((m, k), dtype=np.uint64) if want_polys else None
    codes = np.empty((m, n_lig), dtype=np.uint64) if want_codes else None
    lib().or_encode_rows(_ptr(padded), m, k, n_lig,
                         _ptr(polys) if want_polys else None,
                         _ptr(codes) if want_codes else None)
    return polys, codes


def fold_products_eval(A, B, n_eval, weights=None, ia=None, ib=None):
    """sum_i w[i] * NTT(A[ia[i]] | 0) * NTT(B[ib[i]] | 0) in the n_eval-point domain."""
    A, B = _u64(A), _u64(B)
    k = A.shape[1]
    assert B.shape[1] == k
    if ia is not None:
        ia = np.ascontiguousarray(np.asarray(ia, dtype=np.int64))
        ib = np.ascontiguousarray(np.asarray(ib, dtype=np.int64))
        T = ia.size
    else:
        T = A.shape[0]
    w = None if weights is None else _u64(weights)
    out = np.empty(n_eval, dtype=np.uint64)
    lib().or_fold_products_eval(_ptr(A), A.shape[0], _ptr(B), B.shape[0], k,
                                None if ia is None else _ptr(ia), None if ib is None else _ptr(ib),
                                None if w is None else _ptr(w), T, n_eval, _ptr(out))
    return out


# ---- hashing -----------------------------------------------------------
def blake3(data: bytes) -> bytes:
    buf = np.frombuffer(bytes(data), dtype=np.uint8) if len(data) else np.zeros(1, np.uint8)
    out = np.empty(32, dtype=np.uint8)
    lib().or_blake3(_ptr(np.ascontiguousarray(buf)), len(data), _ptr(out))
    return out.tobytes()


def hash_columns(mat):
    mat = _u64(mat)
    m, n = mat.shape
    out = np.empty((n, 32), dtype=np.uint8)
    lib().or_hash_columns(_ptr(mat), m, n, _ptr(out))
    return out


def merkle_levels(leaves):
    """(n,32) uint8 -> list of per-level (k,32) arrays, leaves first, root last."""
    leaves = np.ascontiguousarray(np.asarray(leaves, dtype=np.uint8))
    n = leaves.shape[0]
    total = lib().or_merkle_total_nodes(n)
    buf = np.empty((total, 32), dtype=np.uint8)
    lib().or_merkle_levels(_ptr(leaves), n, _ptr(buf))
    out, off = [], 0
    while True:
        out.append(buf[off:off + n])
        off += n
        if n <= 1:
            break
        n = (n + 1) // 2
    return out


def merkle_path(levels, idx: int):
    """Opening path of leaf `idx`: per level below the root (sibling bytes, side), the sibling
    being the node itself where an odd level has none, side = 1 when the path node is the left
    child.  Follows merkle_path (prover/core.py:305-317) on the levels of merkle_levels()."""
    path = []
    for level in levels[:-1]:
        sib = idx ^ 1
        if sib >= len(level):
            sib = idx
        path.append((bytes(level[sib].tobytes()), 1 if (idx & 1) == 0 else 0))
        idx //= 2
    return path


def merkle_verify(leaf: bytes, path, root: bytes) -> bool:
    """Recompute the root from a leaf and its path (merkle_verify, prover/core.py:318-323)."""
    cur = leaf
    for sib, side in path:
        cur = blake3(cur + sib) if side == 1 else blake3(sib + cur)
    return cur == root


def row_prg(seed: bytes, row_offset: int, n_rows: int, slack: int):
    s = np.frombuffer(bytes(seed), dtype=np.uint8).copy()
    out = np.empty((n_rows, slack), dtype=np.uint64)
    lib().or_row_prg(_ptr(s), row_offset, n_rows, slack, _ptr(out))
    return out


def row_prg_indexed(seed: bytes, rows, slack: int):
    s = np.frombuffer(bytes(seed), dtype=np.uint8).copy()
    rows = _u64(rows)
    out = np.empty((rows.size, slack), dtype=np.uint64)
    lib().or_row_prg_indexed(_ptr(s), _ptr(rows), rows.size, slack, _ptr(out))
    return out


def challenge(seed: bytes, cid: int, label: bytes = b"") -> int:
    s = np.frombuffer(bytes(seed), dtype=np.uint8).copy()
    lb = np.frombuffer(bytes(label) + b"\0", dtype=np.uint8).copy()
    return lib().or_challenge(_ptr(s), _ptr(lb), len(label), int(cid))


# ---- K-quant -----------------------------------------------------------
QTYPE = {"Q4_K": 4, "Q5_K": 5, "Q6_K": 6}
BLOCK_BYTES = {"Q4_K": 144, "Q5_K": 176, "Q6_K": 210}


def kquant_to_field(raw, qtype: str, S: float):
    raw = np.ascontiguousarray(np.asarray(raw, dtype=np.uint8)).reshape(-1)
    nb = raw.size // BLOCK_BYTES[qtype]
    assert nb * BLOCK_BYTES[qtype] == raw.size
    out = np.empty(nb * 256, dtype=np.uint64)
    rc = lib().or_kquant_to_field(_ptr(raw), nb, QTYPE[qtype], float(S), _ptr(out))
    assert rc == 0
    return out


def signed_to_field(v):
    v = np.ascontiguousarray(np.asarray(v, dtype=np.int64)).reshape(-1)
    out = np.empty(v.size, dtype=np.uint64)
    lib().or_signed_to_field(_ptr(v), v.size, _ptr(out))
    return out


# ---- sumcheck ----------------------------------------------------------
def sumcheck(tables, terms, challenges):
    """tables: (n_tables, size) uint64; terms: [(coef, [table indices])];
    challenges: one per round.  Returns (claim, samples (rounds, deg+1), finals)."""
    tables = _u64(tables)
    nt, size = tables.shape
    n_rounds = size.bit_length() - 1
    max_fac = max(len(f) for _, f in terms)
    coefs = _u64([c % P for c, _ in terms])
    nfac = np.ascontiguousarray(np.array([len(f) for _, f in terms], dtype=np.int32))
    fac = np.zeros((len(terms), max_fac), dtype=np.int32)
    for t, (_, f) in enumerate(terms):
        fac[t, :len(f)] = f
    ch = _u64([c % P for c in challenges])
    assert ch.size == n_rounds
    claim = np.zeros(1, dtype=np.uint64)
    samples = np.zeros((max(n_rounds, 1), max_fac + 1), dtype=np.uint64)
    finals = np.zeros(nt, dtype=np.uint64)
    rc = lib().or_sumcheck(_ptr(tables), nt, size, len(terms), _ptr(coefs), _ptr(nfac),
                           _ptr(fac), max_fac, _ptr(ch), _ptr(claim), _ptr(samples), _ptr(finals))
    assert rc == 0
    return int(claim[0]), samples[:n_rounds], finals


def commit_rows(padded, n_lig) -> bytes:
    padded = _u64(padded)
    m, k = padded.shape
    root = np.empty(32, dtype=np.uint8)
    lib().or_commit_rows(_ptr(padded), m, k, n_lig, _ptr(root))
    return root.tobytes()


def hash_subtree(mat, first_chunk: int):
    """Non-root sub-tree chaining values (ncols, 32) of a block of whole chunks (see verinf_oracle.c)."""
    mat = _u64(mat)
    m, n = mat.shape
    out = np.empty((n, 32), dtype=np.uint8)
    lib().or_hash_subtree(_ptr(mat), m, n, int(first_chunk), _ptr(out))
    return out


def hash_merge_subtrees(cvs, levels):
    cvs = np.ascontiguousarray(np.asarray(cvs, dtype=np.uint8))
    nb, n, _ = cvs.shape
    lv = np.ascontiguousarray(np.asarray(levels, dtype=np.int32))
    out = np.empty((n, 32), dtype=np.uint8)
    rc = lib().or_hash_merge_subtrees(_ptr(cvs), _ptr(lv), nb, n, _ptr(out))
    assert rc == 0
    return out
