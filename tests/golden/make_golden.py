"""Generate the golden fixtures in this directory from the reference's own Python.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's CPU code (prover/ref/goldilocks_ref.py,
prover/protocol.py, layergkr/rs.py, layergkr/sumcheck.py, layergkr/transcript.py)
and the third-party packages the reference itself depends on (`blake3`, `gguf`),
feeds them seeded inputs and stores inputs + outputs as small .npz files.  The
fixtures are what the CPU oracle and the CUDA kernels are pinned against; the
tests never import the reference.
"""
import hashlib
import random
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/reference [fixture ...]")
REF = Path(sys.argv[1]).resolve()
sys.path.insert(0, str(REF))
sys.path.insert(0, str(REF / "prover" / "ref"))

import blake3  # noqa: E402
import goldilocks_ref as gref  # noqa: E402
from prover import protocol  # noqa: E402
from layergkr import rs, sumcheck, transcript  # noqa: E402

P = gref.P


def u64(x):
    return np.array(x, dtype=np.uint64)


def field_vectors():
    """Same cases as goldilocks_ref.emit_field_vectors (seed 42: 11 edge + 50 random)."""
    rng = random.Random(42)
    cases = [(0, 0), (1, 0), (0, 1), (1, 1), (P - 1, 1), (P - 1, P - 1), (0, 1), (1, 2),
             (P - 1, P - 1), (1 << 32, 1 << 32), (1 << 63, 1 << 63)]
    for _ in range(50):
        cases.append((rng.randrange(P), rng.randrange(P)))
    a = [c[0] for c in cases]
    b = [c[1] for c in cases]
    np.savez(HERE / "field_vectors.npz", a=u64(a), b=u64(b),
             add=u64([gref.add(x, y) for x, y in cases]),
             sub=u64([gref.sub(x, y) for x, y in cases]),
             mul=u64([gref.mul(x, y) for x, y in cases]),
             pow12345=u64([pow(x, 12345, P) for x in a]),
             inv=u64([gref.inv(x) if x else 0 for x in a]))


def ntt_vectors():
    """goldilocks_ref.emit_ntt_vectors inputs (seed 123) for several lengths, both directions."""
    out = {}
    for n in (2, 4, 8, 16, 64, 256, 1024, 4096):
        rng = random.Random(123)
        a = [rng.randrange(P) for _ in range(n)]
        w = gref.root_of_unity(n)
        out[f"in_{n}"] = u64(a)
        out[f"fwd_{n}"] = u64(gref.ntt(a, w, invert=False))
        out[f"inv_{n}"] = u64(gref.ntt(a, w, invert=True))
    # Bailey cross-check value the reference keeps for itself (ntt_bailey == ntt)
    rng = random.Random(7)
    a = [rng.randrange(P) for _ in range(1024)]
    assert gref.ntt_bailey(a, 32, 32) == gref.ntt(a, gref.root_of_unity(1024))
    np.savez(HERE / "ntt_vectors.npz", **out)


def encode_vectors():
    """layergkr.rs.encode_row (= protocol.eval_zeta_form) codewords, leaves, Merkle trees."""
    out = {}
    for (ell, k, n, rows, seed) in ((8, 8, 32, 3, 11), (16, 32, 128, 5, 12), (64, 64, 256, 4, 13),
                                    (48, 64, 256, 130, 14)):
        cfg = protocol.Config(ELL=ell, K_DEG=k, N_LIG=n, T_QUERIES=2)
        r = random.Random(seed)
        msgs = [[r.randrange(P) for _ in range(ell)] for _ in range(rows)]
        codes = [rs.encode_row(cfg, m) for m in msgs]
        # spot check against the definition
        for j in (0, 1, n - 1):
            assert codes[0][j] == protocol.eval_zeta_form(cfg, msgs[0], cfg.eta(j))
        com = rs.Commit(cfg, codes)
        tag = f"{ell}_{k}_{n}"
        out[f"msg_{tag}"] = u64(msgs)
        out[f"code_{tag}"] = u64(codes)
        out[f"leaves_{tag}"] = np.frombuffer(b"".join(com.levels[0]), dtype=np.uint8).reshape(-1, 32)
        out[f"root_{tag}"] = np.frombuffer(com.root, dtype=np.uint8)
        out[f"tree_{tag}"] = np.frombuffer(b"".join(b"".join(l) for l in com.levels), dtype=np.uint8)
    np.savez_compressed(HERE / "encode_vectors.npz", **out)


def config1():
    """The reference's CPU-runnable commit case: 64 rows x 2^10 uniform in [0,p) from seed 0, K=2^10, N=2^12,
    column leaves + Merkle root.  The full codeword matrix is 2 MiB, so the fixture keeps
    its sha256, four full rows, 16 full columns, all leaves' sha256 and the root."""
    cfg = protocol.Config(ELL=1024, K_DEG=1024, N_LIG=4096, T_QUERIES=4)
    r = random.Random(0)
    msgs = [[r.randrange(P) for _ in range(1024)] for _ in range(64)]
    codes = [rs.encode_row(cfg, m) for m in msgs]
    com = rs.Commit(cfg, codes)
    mat = u64(codes)
    cols = [0, 1, 2, 3, 255, 256, 1023, 1024, 1025, 2047, 2048, 3000, 4093, 4094, 4095, 13]
    np.savez_compressed(
        HERE / "config1.npz",
        code_sha256=np.frombuffer(hashlib.sha256(mat.tobytes()).digest(), dtype=np.uint8),
        rows_idx=np.array([0, 1, 31, 63]), rows=mat[[0, 1, 31, 63]],
        cols_idx=np.array(cols), cols=mat[:, cols],
        leaves_sha256=np.frombuffer(hashlib.sha256(b"".join(com.levels[0])).digest(), dtype=np.uint8),
        leaves_head=np.frombuffer(b"".join(com.levels[0][:8]), dtype=np.uint8).reshape(-1, 32),
        root=np.frombuffer(com.root, dtype=np.uint8))


def hash_vectors():
    """BLAKE3 known answers (the `blake3` package) + column leaves/trees of odd shapes
    via protocol.merkle_leaf and rs.build_tree + PRF / pad-PRG / transcript values."""
    out = {}
    lengths = [0, 1, 63, 64, 65, 1023, 1024, 1025, 2048, 3072, 4096, 5000, 8192, 16384, 65536]
    out["b3_lengths"] = np.array(lengths)
    out["b3_digests"] = np.frombuffer(
        b"".join(blake3.blake3(bytes(i % 251 for i in range(n))).digest() for n in lengths),
        dtype=np.uint8).reshape(-1, 32)
    r = random.Random(21)
    for (m, n) in ((1, 5), (7, 3), (8, 4), (64, 9), (127, 6), (128, 6), (129, 6), (300, 37),
                   (1024, 5), (1500, 2)):
        mat = [[r.randrange(P) for _ in range(n)] for _ in range(m)]
        leaves = [protocol.merkle_leaf([mat[i][j] for i in range(m)]) for j in range(n)]
        levels = rs.build_tree(leaves)
        out[f"mat_{m}_{n}"] = u64(mat)
        out[f"leaves_{m}_{n}"] = np.frombuffer(b"".join(leaves), dtype=np.uint8).reshape(-1, 32)
        out[f"tree_{m}_{n}"] = np.frombuffer(b"".join(b"".join(l) for l in levels), dtype=np.uint8)
    # challenge PRF (protocol.challenge)
    seed = bytes(range(32))
    cids = [0, 1, 2, 255, 256, 65535, 1 << 32, (1 << 63) + 5]
    for label in ("", "lin", "irs", "quad"):
        out[f"chal_{label or 'none'}"] = u64([protocol.challenge(seed, c, label) for c in cids])
    out["chal_seed"] = np.frombuffer(seed, dtype=np.uint8)
    out["chal_cids"] = u64(cids)
    # pad PRG: formula of cuda_primitives.row_prg's docstring, evaluated with the blake3 package
    rows = [0, 1, 2, 1000, (1 << 32) - 1]
    prg = [[int.from_bytes(blake3.blake3(seed + rr.to_bytes(8, "little") + k.to_bytes(8, "little"))
                           .digest()[:8], "little") % P for k in range(9)] for rr in rows]
    out["prg_rows"] = u64(rows)
    out["prg"] = u64(prg)
    # transcript coins (layergkr.transcript.Transcript)
    t = transcript.Transcript(b"bench/sumcheck")
    t.absorb("seed", (0).to_bytes(8, "little"))
    out["coins_seed0_sc24"] = u64(t.coin("sc", 24))
    np.savez_compressed(HERE / "hash_vectors.npz", **out)


def kquant_vectors():
    """gguf-py dequantize -> round-half-even(double(v) * S) -> signed-to-field, on seeded
    synthetic super-blocks (same composition as prover/tests/test_kquant_kernel.py)."""
    import torch
    from gguf.constants import GGMLQuantizationType as T
    from gguf.quants import dequantize
    rng = np.random.default_rng(5)
    out = {}
    S = 1 << 12
    for name, nbytes, qt in (("Q4_K", 144, T.Q4_K), ("Q5_K", 176, T.Q5_K), ("Q6_K", 210, T.Q6_K)):
        nb = 24
        raw = rng.integers(0, 256, size=(nb, nbytes), dtype=np.uint8)
        # finite f16 scales ~ N(0, 0.02) in the header slots; a few extreme ones too
        d = rng.normal(0, 0.02, size=nb).astype(np.float16)
        dm = rng.normal(0, 0.02, size=nb).astype(np.float16)
        d[0], dm[0] = np.float16(0.0), np.float16(-0.0)
        d[1], dm[1] = np.float16(6.1e-5), np.float16(-5.96e-8)      # subnormal halves
        d[2], dm[2] = np.float16(1.5), np.float16(-2.25)
        if name == "Q6_K":
            raw[:, 208:210] = d.view(np.uint8).reshape(nb, 2)
        else:
            raw[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
            raw[:, 2:4] = dm.view(np.uint8).reshape(nb, 2)
        f = dequantize(raw, qt)                                      # (nb, 256) float32
        assert f.dtype == np.float32 and np.isfinite(f).all()
        ti = torch.round(torch.from_numpy(f.copy()).to(torch.float64) * S).to(torch.int64).numpy()
        field = np.where(ti >= 0, ti, 0).astype(np.uint64)
        neg = ti < 0
        field[neg] = (P - (-ti[neg]).astype(np.uint64).astype(object)).astype(np.uint64) if neg.any() else 0
        out[f"raw_{name}"] = raw
        out[f"field_{name}"] = field.reshape(-1)
    out["S"] = np.array([S])
    np.savez_compressed(HERE / "kquant_vectors.npz", **out)


def sumcheck_vectors():
    """layergkr.sumcheck.prove_terms (pure-Python branch) on seeded instances."""
    out = {}
    r = random.Random(31)
    cases = {
        "deg3_n6": (64, [(1, [0, 1, 2])], 3),
        "deg2_n4": (16, [(1, [0, 1])], 2),
        "terms_n6": (64, [(1, [0, 1]), (P - 1, [0])], 2),
        "mixed_n8": (256, [(5, [0, 1, 2]), (P - 3, [1, 3]), (7, [2])], 4),
        "single_n1": (2, [(1, [0, 1, 2])], 3),
    }
    for name, (size, terms_idx, ntab) in cases.items():
        tabs = [[r.randrange(P) for _ in range(size)] for _ in range(ntab)]
        n_rounds = size.bit_length() - 1
        coins = [r.randrange(P) for _ in range(n_rounds)]
        terms = [(c, [tabs[i] for i in idx]) for c, idx in terms_idx]
        pf = sumcheck.prove_terms(terms, lambda i: coins[i])
        ok, why = sumcheck.verify_terms(pf, terms, lambda i: coins[i])
        assert ok, why
        out[f"{name}_tables"] = u64(tabs)
        out[f"{name}_coins"] = u64(coins)
        out[f"{name}_claim"] = u64([pf.claim])
        out[f"{name}_polys"] = u64([[y for _, y in rp] for rp in pf.round_polys])
        out[f"{name}_terms"] = np.array(
            [[c] + idx + [-1] * (4 - len(idx)) for c, idx in terms_idx], dtype=object).astype(str)
    np.savez_compressed(HERE / "sumcheck_vectors.npz", **out)


def sumcheck_masked_vectors():
    """Masked sumcheck (layergkr/sumcheck.py:192-224): prove_terms with a mask tape and a carried
    mask mu0, pure-Python branch; the cases follow layergkr/tests/test_sumcheck.py:59-68."""
    out = {}
    r = random.Random(47)
    cases = {
        "m_deg2_n4": (16, [(1, [0, 1])], 2),
        "m_deg3_n6": (64, [(1, [0, 1, 2])], 3),
        "m_terms_n8": (256, [(5, [0, 1, 2]), (P - 3, [1, 3]), (7, [2])], 4),
    }
    for name, (size, terms_idx, ntab) in cases.items():
        tabs = [[r.randrange(P) for _ in range(size)] for _ in range(ntab)]
        n_rounds = size.bit_length() - 1
        deg = max(len(idx) for _, idx in terms_idx)
        coins = [r.randrange(P) for _ in range(n_rounds)]
        tape_vals = [r.randrange(P) for _ in range(deg * n_rounds)]
        mu0 = r.randrange(P)
        terms = [(c, [tabs[i] for i in idx]) for c, idx in terms_idx]
        pf = sumcheck.prove_terms(terms, lambda i: coins[i], tape=sumcheck.MaskTape(list(tape_vals)), mu0=mu0)
        ok, why = sumcheck.verify_terms(pf, terms, lambda i: coins[i])
        assert ok, why
        bare = sumcheck.prove_terms(terms, lambda i: coins[i])
        assert pf.claim == (bare.claim + mu0) % P and pf.round_polys[0] != bare.round_polys[0]
        out[f"{name}_tables"] = u64(tabs)
        out[f"{name}_coins"] = u64(coins)
        out[f"{name}_tape"] = u64(tape_vals)
        out[f"{name}_mu0"] = u64([mu0])
        out[f"{name}_claim"] = u64([pf.claim])
        out[f"{name}_final_mask"] = u64([pf.final_mask])
        out[f"{name}_polys"] = u64([[y for _, y in rp] for rp in pf.round_polys])
        out[f"{name}_terms"] = np.array(
            [[c] + idx + [-1] * (4 - len(idx)) for c, idx in terms_idx], dtype=object).astype(str)
    np.savez_compressed(HERE / "sumcheck_masked_vectors.npz", **out)


def merkle_path_vectors():
    """Opening paths from rs.build_tree + rs.merkle_path (same convention as
    prover/core.merkle_path) for every leaf of trees with 1, 2, 5, 8 and 13 leaves; each path is
    checked with protocol.merkle_verify before it is stored."""
    rng = random.Random(2024)
    out = {}
    for n in (1, 2, 5, 8, 13):
        leaves = [bytes(rng.randrange(256) for _ in range(32)) for _ in range(n)]
        levels = rs.build_tree(leaves)
        depth = len(levels) - 1
        sib = np.zeros((n, depth, 32), dtype=np.uint8)
        side = np.zeros((n, depth), dtype=np.uint8)
        for i in range(n):
            path = rs.merkle_path(levels, i)
            assert protocol.merkle_verify(leaves[i], path, levels[-1][0])
            for l, (s, d) in enumerate(path):
                sib[i, l] = np.frombuffer(s, dtype=np.uint8)
                side[i, l] = d
        out[f"n{n}_leaves"] = np.frombuffer(b"".join(leaves), dtype=np.uint8).reshape(n, 32)
        out[f"n{n}_root"] = np.frombuffer(levels[-1][0], dtype=np.uint8)
        out[f"n{n}_siblings"] = sib
        out[f"n{n}_sides"] = side
    np.savez_compressed(HERE / "merkle_path_vectors.npz", **out)


def fold_vectors():
    """Evaluation-domain fold of row products built from the reference's own CPU NTT and field
    ops (goldilocks_ref.ntt / mul / add), following the data flow of the fused q_lin branch
    (prover/core.py:1892-1911) and of compute_p_0_streaming's weighted_eval (:2166-2181):
    zero-extend to n_eval = next_pow2(2K-1), forward NTT both factors, multiply pointwise,
    weighted sum over the rows.  Also stores the inverse transform cut to 2K-1 coefficients and
    checks it against schoolbook polynomial products."""
    rng = random.Random(77)
    out = {}
    for name, m, K, T in (("small", 5, 16, 5), ("indexed", 6, 32, 11)):
        n_eval = 1
        while n_eval < 2 * K - 1:
            n_eval <<= 1
        A = [[rng.randrange(P) for _ in range(K)] for _ in range(m)]
        B = [[rng.randrange(P) for _ in range(K)] for _ in range(m)]
        w = [rng.randrange(P) for _ in range(T)]
        ia = list(range(m)) if T == m else [rng.randrange(m) for _ in range(T)]
        ib = list(range(m)) if T == m else [rng.randrange(m) for _ in range(T)]
        om = gref.root_of_unity(n_eval)
        EA = [gref.ntt(row + [0] * (n_eval - K), om) for row in A]
        EB = [gref.ntt(row + [0] * (n_eval - K), om) for row in B]
        ev_w = [0] * n_eval
        ev_1 = [0] * n_eval
        for t in range(T):
            for j in range(n_eval):
                pr = gref.mul(EA[ia[t]][j], EB[ib[t]][j])
                ev_1[j] = gref.add(ev_1[j], pr)
                ev_w[j] = gref.add(ev_w[j], gref.mul(pr, w[t]))
        coef = gref.ntt(ev_w, om, invert=True)
        want = [0] * n_eval
        for t in range(T):
            for x in range(K):
                for y in range(K):
                    want[x + y] = (want[x + y] + w[t] * A[ia[t]][x] * B[ib[t]][y]) % P
        assert coef == want and coef[2 * K - 1:] == [0] * (n_eval - 2 * K + 1)
        out[f"{name}_A"] = u64(A); out[f"{name}_B"] = u64(B); out[f"{name}_w"] = u64(w)
        out[f"{name}_ia"] = np.array(ia, dtype=np.int64); out[f"{name}_ib"] = np.array(ib, dtype=np.int64)
        out[f"{name}_eval_weighted"] = u64(ev_w); out[f"{name}_eval_ones"] = u64(ev_1)
        out[f"{name}_coef"] = u64(coef[:2 * K - 1])
    np.savez_compressed(HERE / "fold_vectors.npz", **out)


if __name__ == "__main__":
    if len(sys.argv) > 2:                                         # only the named fixtures
        for name in sys.argv[2:]:
            {"merkle_paths": merkle_path_vectors, "fold": fold_vectors,
             "sumcheck_masked": sumcheck_masked_vectors}[name]()
        sys.exit(0)
    fold_vectors()
    merkle_path_vectors()
    field_vectors()
    ntt_vectors()
    hash_vectors()
    kquant_vectors()
    sumcheck_vectors()
    sumcheck_masked_vectors()
    encode_vectors()
    config1()
    print("golden fixtures written to", HERE)
