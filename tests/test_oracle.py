"""CPU: the C oracle against the golden fixtures made from the reference's own Python."""
import hashlib

import numpy as np
import pytest

import oracle

P = oracle.P


def test_field_vectors(golden):
    g = golden.field_vectors
    for a, b, s, d, m, pw, iv in zip(g["a"], g["b"], g["add"], g["sub"], g["mul"], g["pow12345"], g["inv"]):
        a, b = int(a), int(b)
        assert oracle.gl_add(a, b) == int(s)
        assert oracle.gl_sub(a, b) == int(d)
        assert oracle.gl_mul(a, b) == int(m)
        assert oracle.gl_pow(a, 12345) == int(pw)
        if a:
            assert oracle.gl_inv(a) == int(iv)


@pytest.mark.parametrize("n", [2, 4, 8, 16, 64, 256, 1024, 4096])
def test_ntt_vectors(golden, n):
    g = golden.ntt_vectors
    x = g[f"in_{n}"]
    assert np.array_equal(oracle.ntt(x), g[f"fwd_{n}"])
    assert np.array_equal(oracle.ntt(x, invert=True), g[f"inv_{n}"])
    rows = np.stack([x, g[f"fwd_{n}"]])
    assert np.array_equal(oracle.ntt_batched(rows)[0], g[f"fwd_{n}"])
    assert np.array_equal(oracle.ntt_batched(rows, invert=True)[1], x)


@pytest.mark.parametrize("tag", ["8_8_32", "16_32_128", "64_64_256", "48_64_256"])
def test_encode_and_commit_vectors(golden, tag):
    g = golden.encode_vectors
    ell, k, n = (int(v) for v in tag.split("_"))
    msg = g[f"msg_{tag}"]
    padded = np.zeros((msg.shape[0], k), dtype=np.uint64)
    padded[:, :ell] = msg
    polys, codes = oracle.encode_rows(padded, n)
    assert np.array_equal(codes, g[f"code_{tag}"])
    assert np.array_equal(oracle.ntt_batched(polys), padded)
    leaves = oracle.hash_columns(codes)
    assert np.array_equal(leaves, g[f"leaves_{tag}"])
    levels = oracle.merkle_levels(leaves)
    assert levels[-1].tobytes() == g[f"root_{tag}"].tobytes()
    assert b"".join(l.tobytes() for l in levels) == g[f"tree_{tag}"].tobytes()
    assert oracle.commit_rows(padded, n) == g[f"root_{tag}"].tobytes()


def test_config1(golden):
    import random
    g = golden.config1
    r = random.Random(0)
    msg = np.array([[r.randrange(P) for _ in range(1024)] for _ in range(64)], dtype=np.uint64)
    _, codes = oracle.encode_rows(msg, 4096, want_polys=False)
    assert hashlib.sha256(codes.tobytes()).digest() == g["code_sha256"].tobytes()
    assert np.array_equal(codes[g["rows_idx"]], g["rows"])
    assert np.array_equal(codes[:, g["cols_idx"]], g["cols"])
    leaves = oracle.hash_columns(codes)
    assert hashlib.sha256(leaves.tobytes()).digest() == g["leaves_sha256"].tobytes()
    assert np.array_equal(leaves[:8], g["leaves_head"])
    assert oracle.merkle_levels(leaves)[-1].tobytes() == g["root"].tobytes()


def test_blake3_and_column_trees(golden):
    g = golden.hash_vectors
    for n, d in zip(g["b3_lengths"], g["b3_digests"]):
        assert oracle.blake3(bytes(i % 251 for i in range(int(n)))) == d.tobytes()
    for key in g.files:
        if not key.startswith("mat_"):
            continue
        tag = key[4:]
        leaves = oracle.hash_columns(g[key])
        assert np.array_equal(leaves, g[f"leaves_{tag}"]), tag
        assert b"".join(l.tobytes() for l in oracle.merkle_levels(leaves)) == g[f"tree_{tag}"].tobytes(), tag


def test_prf_prg_coins(golden):
    g = golden.hash_vectors
    seed = g["chal_seed"].tobytes()
    for label in ("", "lin", "irs", "quad"):
        want = g[f"chal_{label or 'none'}"]
        got = [oracle.challenge(seed, int(c), label.encode()) for c in g["chal_cids"]]
        assert got == [int(v) for v in want]
    assert np.array_equal(oracle.row_prg_indexed(seed, g["prg_rows"], 9), g["prg"])
    assert np.array_equal(oracle.row_prg(seed, 0, 3, 9), g["prg"][:3])


@pytest.mark.parametrize("qt", ["Q4_K", "Q5_K", "Q6_K"])
def test_kquant_vectors(golden, qt):
    g = golden.kquant_vectors
    got = oracle.kquant_to_field(g[f"raw_{qt}"], qt, float(g["S"][0]))
    assert np.array_equal(got, g[f"field_{qt}"])


@pytest.mark.parametrize("name", ["deg3_n6", "deg2_n4", "terms_n6", "mixed_n8", "single_n1"])
def test_sumcheck_vectors(golden, name):
    g = golden.sumcheck_vectors
    terms = []
    for row in g[f"{name}_terms"]:
        vals = [int(v) for v in row]
        terms.append((vals[0], [v for v in vals[1:] if v >= 0]))
    claim, samples, _ = oracle.sumcheck(g[f"{name}_tables"], terms, [int(c) for c in g[f"{name}_coins"]])
    assert claim == int(g[f"{name}_claim"][0])
    want = g[f"{name}_polys"]
    assert np.array_equal(samples[:, :want.shape[1]], want)


@pytest.mark.parametrize("name", ["m_deg2_n4", "m_deg3_n6", "m_terms_n8"])
def test_sumcheck_masked_vectors(golden, name):
    """Oracle samples plus the scalar mask of layergkr/sumcheck.py:192-224 reproduce the
    reference's masked transcript (the mask never touches the tables)."""
    g = golden.sumcheck_masked_vectors
    terms = []
    for row in g[f"{name}_terms"]:
        vals = [int(v) for v in row]
        terms.append((vals[0], [v for v in vals[1:] if v >= 0]))
    coins = [int(c) for c in g[f"{name}_coins"]]
    tape = [int(v) for v in g[f"{name}_tape"]]
    claim, samples, _ = oracle.sumcheck(g[f"{name}_tables"], terms, coins)
    deg = max(len(f) for _, f in terms)
    mu = int(g[f"{name}_mu0"][0])
    assert (claim + mu) % oracle.P == int(g[f"{name}_claim"][0])
    inv2 = pow(2, oracle.P - 2, oracle.P)
    ev = lambda h, x: sum(c * pow(x, i, oracle.P) for i, c in enumerate(h)) % oracle.P
    for rnd, r in enumerate(coins):
        u = tape[rnd * deg:(rnd + 1) * deg]
        h = [((mu - sum(u)) % oracle.P) * inv2 % oracle.P] + u
        got = [(int(samples[rnd][x]) + ev(h, x)) % oracle.P for x in range(deg + 1)]
        assert got == [int(v) for v in g[f"{name}_polys"][rnd]]
        mu = ev(h, r)
    assert mu == int(g[f"{name}_final_mask"][0])


@pytest.mark.parametrize("n", [1, 2, 5, 8, 13])
def test_merkle_path_vectors(golden, n):
    g = golden.merkle_path_vectors
    leaves = g[f"n{n}_leaves"]
    levels = oracle.merkle_levels(leaves)
    root = g[f"n{n}_root"].tobytes()
    assert levels[-1][0].tobytes() == root
    for i in range(n):
        path = oracle.merkle_path(levels, i)
        assert [s for s, _ in path] == [g[f"n{n}_siblings"][i, l].tobytes() for l in range(len(path))]
        assert [d for _, d in path] == [int(v) for v in g[f"n{n}_sides"][i]]
        assert oracle.merkle_verify(leaves[i].tobytes(), path, root)
        assert n == 1 or not oracle.merkle_verify(leaves[(i + 1) % n].tobytes(), path, root)


def test_matmul_against_python_integers():
    rng = np.random.default_rng(12)
    A = rng.integers(0, P, size=(5, 37), dtype=np.uint64)
    B = rng.integers(0, P, size=(37, 4), dtype=np.uint64)
    A[0, :] = P - 1
    B[:, 0] = P - 1
    got = oracle.gl_matmul(A, B)
    for i in range(5):
        for j in range(4):
            assert int(got[i, j]) == sum(int(A[i, l]) * int(B[l, j]) for l in range(37)) % P


@pytest.mark.parametrize("name", ["small", "indexed"])
def test_fold_vectors(golden, name):
    g = golden.fold_vectors
    A, B, w, ia, ib = (g[f"{name}_{k}"] for k in ("A", "B", "w", "ia", "ib"))
    n_eval = g[f"{name}_eval_ones"].size
    assert np.array_equal(oracle.fold_products_eval(A, B, n_eval, w, ia, ib), g[f"{name}_eval_weighted"])
    assert np.array_equal(oracle.fold_products_eval(A, B, n_eval, None, ia, ib), g[f"{name}_eval_ones"])
    coef = oracle.ntt(oracle.fold_products_eval(A, B, n_eval, w, ia, ib), invert=True)
    assert np.array_equal(coef[:g[f"{name}_coef"].size], g[f"{name}_coef"]) and not coef[g[f"{name}_coef"].size:].any()
    if name == "small":
        assert np.array_equal(oracle.fold_products_eval(A, B, n_eval, w), g[f"{name}_eval_weighted"])
