"""GPU parity: the CUDA path (through the C ABI, via the drop-in modules) against the CPU
oracle and the golden fixtures.  Integer work: every comparison is bit-exact."""
import hashlib
import random

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle  # noqa: E402

P = oracle.P


@pytest.fixture(scope="module")
def cp():
    from verinf_b200 import cuda_primitives
    return cuda_primitives


def dev(a):
    a = np.ascontiguousarray(np.asarray(a, dtype=np.uint64))
    return torch.from_numpy(a.view(np.int64)).cuda().view(torch.uint64)


def host(t):
    return t.contiguous().view(torch.int64).cpu().numpy().view(np.uint64)


def rnd_field(rng, shape):
    """uniform in [0, p) by rejection (p is within 2^-32 of 2^64)"""
    a = rng.integers(0, 2**64, size=shape, dtype=np.uint64)
    bad = a >= np.uint64(P)
    while bad.any():
        a[bad] = rng.integers(0, 2**64, size=int(bad.sum()), dtype=np.uint64)
        bad = a >= np.uint64(P)
    return a


# ---------------------------------------------------------------- field ------
def test_field_golden(cp, golden):
    g = golden.field_vectors
    a, b = dev(g["a"]), dev(g["b"])
    assert np.array_equal(host(cp.gl_add(a, b)), g["add"])
    assert np.array_equal(host(cp.gl_sub(a, b)), g["sub"])
    assert np.array_equal(host(cp.gl_mul(a, b)), g["mul"])
    assert np.array_equal(host(cp.gl_pow(a, 12345)), g["pow12345"])
    nz = g["a"] != 0
    assert np.array_equal(host(cp.gl_inv(a))[nz], g["inv"][nz])
    assert np.array_equal(host(cp.gl_inv_batched(a))[nz], g["inv"][nz])
    assert np.array_equal(host(cp.gl_neg(a)), np.array([(P - int(x)) % P for x in g["a"]], dtype=np.uint64))


def test_field_random_and_axpy(cp):
    rng = np.random.default_rng(1)
    n = 100003
    a, b = rnd_field(rng, n), rnd_field(rng, n)
    ai, bi = [int(x) for x in a[:2000]], [int(x) for x in b[:2000]]
    got = host(cp.gl_mul(dev(a), dev(b)))
    assert [int(x) for x in got[:2000]] == [x * y % P for x, y in zip(ai, bi)]
    # whole array through linearity: (a*b) + (a*(p-b)) == 0
    nb = np.where(b == 0, b, np.uint64(P) - b)
    s = cp.gl_add(cp.gl_mul(dev(a), dev(b)), cp.gl_mul(dev(a), dev(nb)))
    assert not host(s).any()
    y, x, alpha = dev(a), dev(b), 0x123456789ABCDEF
    cp.gl_axpy(y, alpha, x)
    assert [int(v) for v in host(y)[:2000]] == [(p + alpha * q) % P for p, q in zip(ai, bi)]
    v = rnd_field(rng, 257)
    m = rnd_field(rng, (5, 257))
    got = host(cp.gl_mul_rowvec(dev(m), dev(v)))
    assert [int(t) for t in got[3]] == [int(p) * int(q) % P for p, q in zip(m[3], v)]
    assert cp.gl_mul(dev(a[:0]), dev(b[:0])).numel() == 0


# ---------------------------------------------------------------- NTT --------
@pytest.mark.parametrize("n", [2, 4, 8, 16, 64, 256, 1024, 4096])
def test_ntt_golden(cp, golden, n):
    g = golden.ntt_vectors
    x = dev(g[f"in_{n}"])
    cp.ntt_forward(x)
    assert np.array_equal(host(x), g[f"fwd_{n}"])
    cp.ntt_inverse(x)
    assert np.array_equal(host(x), g[f"in_{n}"])
    y = dev(g[f"in_{n}"])
    cp.ntt_inverse(y)
    assert np.array_equal(host(y), g[f"inv_{n}"])


@pytest.mark.parametrize("logn", list(range(1, 15)) + [16, 17, 18])
@pytest.mark.parametrize("m", [1, 3, 129])
def test_ntt_batched_vs_oracle(cp, logn, m):
    if logn >= 16 and m == 129:
        m = 17
    rng = np.random.default_rng(100 + logn)
    n = 1 << logn
    a = rnd_field(rng, (m, n))
    x = dev(a)
    cp.ntt_forward_batched(x)
    assert np.array_equal(host(x), oracle.ntt_batched(a))
    cp.ntt_inverse_batched(x)
    assert np.array_equal(host(x), a)
    y = dev(a)
    cp.ntt_inverse_batched(y)
    assert np.array_equal(host(y), oracle.ntt_batched(a, invert=True))


@pytest.mark.parametrize("logn,m", [(25, 2), (26, 1)])
def test_ntt_three_pass(cp, logn, m):
    """Lengths above 2^24 (three tile passes, split four-step factor tables; the reference's dispatch
    takes any power of two, prover/kernels/ntt.cuh:746-770): the whole transform of the last row against
    the oracle, a sparse input against the closed form X[k] = sum_i v_i w_n^(j_i k) at sampled k (first
    row), and the inverse round trip."""
    n = 1 << logn
    rng = np.random.default_rng(logn)
    a = rnd_field(rng, (m, n))
    x = dev(a)
    cp.ntt_forward_batched(x)
    assert np.array_equal(host(x)[m - 1], oracle.ntt(a[m - 1]))
    cp.ntt_inverse_batched(x)
    assert np.array_equal(host(x), a)
    w = pow(7, (P - 1) // n, P)
    pos = [0, 1, n // 3, n - 1, (5 << (logn - 3)) + 77]
    vals = [int(v) for v in rnd_field(rng, len(pos))]
    sp = np.zeros((1, n), dtype=np.uint64)
    for j, v in zip(pos, vals):
        sp[0, j] = v
    y = dev(sp)
    cp.ntt_forward_batched(y)
    got = host(y)[0]
    for k in [0, 1, 2, n // 2, n - 1] + [int(t) for t in rng.integers(0, n, size=200)]:
        assert int(got[k]) == sum(v * pow(w, (j * k) % n, P) for j, v in zip(pos, vals)) % P, k


def test_ntt_large_roundtrip_and_errors(cp):
    rng = np.random.default_rng(7)
    for logn, m in ((20, 2), (21, 1), (22, 2), (24, 1)):
        a = rnd_field(rng, (m, 1 << logn))
        x = dev(a)
        cp.ntt_forward_batched(x)
        assert np.array_equal(host(x)[m - 1], oracle.ntt(a[m - 1])), logn
        cp.ntt_inverse_batched(x)
        assert np.array_equal(host(x), a), logn
    with pytest.raises(RuntimeError):
        cp.ntt_forward(dev(np.arange(12)))
    with pytest.raises(RuntimeError):
        cp.ntt_forward(dev(np.arange(16))[::2])
    with pytest.raises(RuntimeError):
        cp.ntt_forward(torch.zeros(16, dtype=torch.int64, device="cuda"))
    e = torch.empty((0, 64), dtype=torch.uint64, device="cuda")
    cp.ntt_forward_batched(e)


def test_poly_ops(cp):
    rng = np.random.default_rng(9)
    a, b = rnd_field(rng, 37), rnd_field(rng, 90)
    want = [0] * (37 + 90 - 1)
    for i, x in enumerate(a):
        for j, y in enumerate(b):
            want[i + j] = (want[i + j] + int(x) * int(y)) % P
    assert [int(v) for v in host(cp.poly_mul(dev(a), dev(b)))] == want
    A, B = rnd_field(rng, (3, 40)), rnd_field(rng, (3, 40))
    got = host(cp.poly_mul_batched(dev(A), dev(B)))
    assert np.array_equal(got[1], host(cp.poly_mul(dev(A[1]), dev(B[1]))))
    s = host(cp.poly_add(dev(a), dev(b)))
    assert [int(v) for v in s[:37]] == [(int(x) + int(y)) % P for x, y in zip(a, b[:37])]
    pts = rnd_field(rng, 11)
    ev = host(cp.poly_eval(dev(a), dev(pts)))
    for p_, e_ in zip(pts, ev):
        acc = 0
        for c in reversed(a):
            acc = (acc * int(p_) + int(c)) % P
        assert acc == int(e_)
    assert host(cp.poly_eval(dev(A), dev(pts))).shape == (3, 11)


# ---------------------------------------------------------------- encode -----
@pytest.mark.parametrize("tag", ["8_8_32", "16_32_128", "64_64_256", "48_64_256"])
def test_encode_golden(cp, golden, tag):
    g = golden.encode_vectors
    ell, k, n = (int(v) for v in tag.split("_"))
    polys, codes = cp.encode_rows(dev(g[f"msg_{tag}"]), k, n)
    assert np.array_equal(host(codes), g[f"code_{tag}"])
    back = polys.clone()
    cp.ntt_forward_batched(back)
    assert np.array_equal(host(back)[:, :ell], g[f"msg_{tag}"])
    assert not host(back)[:, ell:].any()
    leaves = cp.hash_columns_streamed(codes)
    assert np.array_equal(leaves.cpu().numpy(), g[f"leaves_{tag}"])
    root, levels = cp.merkle_build_blake3(leaves)
    assert root.cpu().numpy().tobytes() == g[f"root_{tag}"].tobytes()
    assert b"".join(l.cpu().numpy().tobytes() for l in levels) == g[f"tree_{tag}"].tobytes()
    assert levels[0] is leaves and tuple(levels[-1].shape) == (1, 32)


def test_config1_golden(cp, golden):
    g = golden.config1
    r = random.Random(0)
    msg = np.array([[r.randrange(P) for _ in range(1024)] for _ in range(64)], dtype=np.uint64)
    root, levels, codes = cp.commit_rows(dev(msg), 1024, 4096)
    c = host(codes)
    assert hashlib.sha256(c.tobytes()).digest() == g["code_sha256"].tobytes()
    assert np.array_equal(c[g["rows_idx"]], g["rows"])
    assert np.array_equal(c[:, g["cols_idx"]], g["cols"])
    assert hashlib.sha256(levels[0].cpu().numpy().tobytes()).digest() == g["leaves_sha256"].tobytes()
    assert root.cpu().numpy().tobytes() == g["root"].tobytes()
    assert len(levels) == 13


ENC_CASES = [(2, 2, 2, 3), (1, 2, 8, 2), (3, 4, 16, 5), (8, 8, 8, 1), (20, 32, 64, 7), (64, 128, 512, 130),
             (512, 512, 2048, 9), (1000, 1024, 4096, 4), (2048, 2048, 4096, 3), (8192, 16384, 65536, 5),
             (30000, 32768, 65536, 2), (65536, 65536, 262144, 3)]


@pytest.mark.parametrize("ell,k,n,m", ENC_CASES)
@pytest.mark.parametrize("pad", [False, True])
def test_encode_vs_oracle(cp, ell, k, n, m, pad):
    rng = np.random.default_rng(ell * 7 + k + m)
    msg = rnd_field(rng, (m, ell))
    seed = bytes(rng.integers(0, 256, size=32, dtype=np.uint8))
    row_off = 1000003
    padded = np.zeros((m, k), dtype=np.uint64)
    padded[:, :ell] = msg
    if pad and ell < k:
        padded[:, ell:] = oracle.row_prg(seed, row_off, m, k - ell)
    want_p, want_c = oracle.encode_rows(padded, n)
    seed_t = torch.tensor(list(seed), dtype=torch.uint8, device="cuda") if pad else None
    polys, codes = cp.encode_rows(dev(msg), k, n, master_seed=seed_t, row_offset=row_off)
    assert np.array_equal(host(polys), want_p)
    assert np.array_equal(host(codes), want_c)
    p2, c2 = cp.encode_rows(dev(msg), k, n, master_seed=seed_t, row_offset=row_off, need_codewords=False)
    assert c2 is None and np.array_equal(host(p2), want_p)
    # same as the reference's unfused pipeline on the primitives
    if pad and ell < k:
        full = dev(padded)
        cp.ntt_inverse_batched(full)
        g = dev(np.array([pow(7, l, P) for l in range(k)], dtype=np.uint64)) if k <= 4096 else None
        if g is not None:
            ext = torch.zeros((m, n), dtype=torch.uint64, device="cuda")
            ext[:, :k] = cp.gl_mul_rowvec(full, g)
            cp.ntt_forward_batched(ext)
            assert torch.equal(ext.view(torch.int64), codes.view(torch.int64))


@pytest.mark.parametrize("ell,k,n,m", [((1 << 21) - 5, 1 << 21, 1 << 22, 2), (1 << 23, 1 << 23, 1 << 24, 1)])
def test_encode_long_rows(cp, ell, k, n, m):
    """K above 2^20: tile DFT lengths 2048 and 4096 (4 and 2 columns per tile)"""
    rng = np.random.default_rng(k % 1009)
    msg = rnd_field(rng, (m, ell))
    seed = bytes(rng.integers(0, 256, size=32, dtype=np.uint8))
    padded = np.zeros((m, k), dtype=np.uint64)
    padded[:, :ell] = msg
    if ell < k:
        padded[:, ell:] = oracle.row_prg(seed, 5, m, k - ell)
    want_p, want_c = oracle.encode_rows(padded, n)
    seed_t = torch.tensor(list(seed), dtype=torch.uint8, device="cuda")
    polys, codes = cp.encode_rows(dev(msg), k, n, master_seed=seed_t, row_offset=5)
    assert np.array_equal(host(polys), want_p)
    assert np.array_equal(host(codes), want_c)


def test_encode_edge_cases(cp):
    e = torch.empty((0, 8), dtype=torch.uint64, device="cuda")
    p, c = cp.encode_rows(e, 8, 32)
    assert tuple(p.shape) == (0, 8) and tuple(c.shape) == (0, 32)
    with pytest.raises(RuntimeError):
        cp.encode_rows(torch.zeros((2, 9), dtype=torch.uint64, device="cuda"), 8, 32)   # ELL > K
    with pytest.raises(RuntimeError):
        cp.encode_rows(torch.zeros((2, 8), dtype=torch.uint64, device="cuda"), 12, 48)  # K not a power of 2
    rng = np.random.default_rng(3)
    msgs = rnd_field(rng, (6, 32))
    out = host(cp.rs_encode_rows(dev(msgs), 128, 32))
    for i in range(6):
        co = oracle.ntt(msgs[i], invert=True)
        ext = np.zeros(128, dtype=np.uint64)
        ext[:32] = co
        assert np.array_equal(out[i], oracle.ntt(ext))


def test_encode_chunking_invariant(cp):
    """small scratch (one row per chunk) and large scratch give identical codewords"""
    from verinf_b200._lib import LIB, check, ptr, stream_ptr
    rng = np.random.default_rng(17)
    m, ell, k, n = 11, 3000, 4096, 16384
    msg = dev(rnd_field(rng, (m, ell)))
    _, want = cp.encode_rows(msg, k, n, need_polys=False)
    codes = torch.empty((m, n), dtype=torch.uint64, device="cuda")
    small = torch.empty(((k + n) * 8,), dtype=torch.uint8, device="cuda")
    check(LIB.vi_encode_rows(ptr(msg), m, ell, k, n, 0, None, 0, None, ptr(codes), ptr(small), small.numel(),
                             stream_ptr()))
    assert torch.equal(codes.view(torch.int64), want.view(torch.int64))
    rc = LIB.vi_encode_rows(ptr(msg), m, ell, k, n, 0, None, 0, None, ptr(codes), ptr(small), 100, stream_ptr())
    assert rc != 0 and b"scratch" in LIB.vi_last_error()


# ---------------------------------------------------------------- hashing ----
def test_hash_golden(cp, golden):
    g = golden.hash_vectors
    for key in g.files:
        if not key.startswith("mat_"):
            continue
        tag = key[4:]
        leaves = cp.hash_columns_streamed(dev(g[key]))
        assert np.array_equal(leaves.cpu().numpy(), g[f"leaves_{tag}"]), tag
        _, levels = cp.merkle_build_blake3(leaves)
        assert b"".join(l.cpu().numpy().tobytes() for l in levels) == g[f"tree_{tag}"].tobytes(), tag


@pytest.mark.parametrize("m,n", [(1, 1), (5, 33), (128, 100), (129, 100), (255, 7), (256, 64), (257, 64),
                                 (1000, 300), (4096, 64), (4224, 40), (16385, 9)])
def test_hash_columns_vs_oracle(cp, m, n):
    rng = np.random.default_rng(m * 31 + n)
    a = rnd_field(rng, (m, n))
    assert np.array_equal(cp.hash_columns_streamed(dev(a)).cpu().numpy(), oracle.hash_columns(a))


@pytest.mark.parametrize("total,pieces", [(129, [129]), (129, [1, 128]), (300, [3, 128, 169]),
                                           (1027, [3, 1024]), (2048, [1024, 1024]), (2051, [3, 1000, 24, 1024]),
                                           (640, [127, 1, 1, 127, 128, 256])])
def test_merkle_column_accumulator(cp, total, pieces):
    assert sum(pieces) == total
    rng = np.random.default_rng(total)
    n = 77
    a = rnd_field(rng, (total, n))
    acc = cp.MerkleColumnAccumulator(n, total)
    t = dev(a)
    off = 0
    for k in pieces:
        acc.update(t[off:off + k])
        off += k
    acc.update(t[:0])
    assert np.array_equal(acc.finalize().cpu().numpy(), oracle.hash_columns(a))
    with pytest.raises(AssertionError):
        cp.MerkleColumnAccumulator(n, 128)


@pytest.mark.parametrize("n", [1, 2, 3, 5, 8, 1000, 1024, 4097])
def test_merkle_vs_oracle(cp, n):
    rng = np.random.default_rng(n)
    leaves = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    root, levels = cp.merkle_build_blake3(torch.from_numpy(leaves).cuda())
    want = oracle.merkle_levels(leaves)
    assert len(levels) == len(want)
    for a, b in zip(levels, want):
        assert np.array_equal(a.cpu().numpy(), b)
    assert root.cpu().numpy().tobytes() == want[-1].tobytes()
    if n % 2 == 0 and n >= 2:
        one = cp._ensure_compiled().merkle_one_level(torch.from_numpy(leaves).cuda().view(torch.uint32))
        assert np.array_equal(one.view(torch.uint8).cpu().numpy(), want[1])


def test_prg_and_challenge(cp, golden):
    g = golden.hash_vectors
    seed = torch.from_numpy(g["chal_seed"].copy()).cuda()
    got = cp.row_prg_indexed(seed, dev(g["prg_rows"]), 9)
    assert np.array_equal(host(got), g["prg"])
    assert np.array_equal(host(cp.row_prg(seed, 0, 3, 9)), g["prg"][:3])
    assert np.array_equal(host(cp.row_prg(seed, 1000, 1, 9)), g["prg"][3:4])
    assert tuple(cp.row_prg(seed, 0, 0, 9).shape) == (0, 9) and tuple(cp.row_prg(seed, 0, 4, 0).shape) == (4, 0)
    big = host(cp.row_prg(seed, 5, 37, 1000))
    assert np.array_equal(big, oracle.row_prg(g["chal_seed"].tobytes(), 5, 37, 1000))
    for label in ("", "lin", "irs", "quad"):
        lab = torch.tensor(list(label.encode()), dtype=torch.uint8, device="cuda")
        got = cp.challenge_at(seed, lab, dev(g["chal_cids"]))
        assert np.array_equal(host(got), g[f"chal_{label or 'none'}"])
        vec = host(cp.challenge_vec(seed, lab, 300))
        assert [int(v) for v in vec[:3]] == [int(v) for v in g[f"chal_{label or 'none'}"][:3]]
        assert int(vec[255]) == int(g[f"chal_{label or 'none'}"][3])
    lab8 = torch.tensor(list(b"abcdefgh"), dtype=torch.uint8, device="cuda")
    v = host(cp.challenge_vec(seed, lab8, 5))
    assert [int(x) for x in v] == [oracle.challenge(g["chal_seed"].tobytes(), i, b"abcdefgh") for i in range(5)]
    assert cp.challenge_vec(seed, lab8, 0).numel() == 0


# ---------------------------------------------------------------- K-quant ----
@pytest.mark.parametrize("qt", ["Q4_K", "Q5_K", "Q6_K"])
def test_kquant_golden_and_oracle(golden, qt):
    from verinf_b200 import kquant_cuda as kq
    g = golden.kquant_vectors
    S = int(g["S"][0])
    got = kq.kquant_to_field(torch.from_numpy(g[f"raw_{qt}"].copy()).cuda(), qt, S)
    assert np.array_equal(host(got), g[f"field_{qt}"])
    rng = np.random.default_rng(11)
    nb = 3001
    raw = synth_blocks(rng, qt, nb)
    got = kq.kquant_to_field(torch.from_numpy(raw).cuda(), qt, S)
    assert np.array_equal(host(got), oracle.kquant_to_field(raw, qt, S))
    assert kq.kquant_to_field(torch.empty(0, dtype=torch.uint8, device="cuda"), qt, S).numel() == 0
    with pytest.raises(RuntimeError):
        kq.kquant_to_field(torch.zeros(100, dtype=torch.uint8, device="cuda"), qt, S)


def synth_blocks(rng, qt, nb):
    nbytes = oracle.BLOCK_BYTES[qt]
    raw = rng.integers(0, 256, size=(nb, nbytes), dtype=np.uint8)
    d = np.clip(rng.normal(0, 0.02, size=nb), -6e4, 6e4).astype(np.float16)
    dm = np.clip(rng.normal(0, 0.02, size=nb), -6e4, 6e4).astype(np.float16)
    if qt == "Q6_K":
        raw[:, 208:210] = d.view(np.uint8).reshape(nb, 2)
    else:
        raw[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
        raw[:, 2:4] = dm.view(np.uint8).reshape(nb, 2)
    return raw


@pytest.mark.parametrize("qt", ["Q4_K", "Q6_K"])
@pytest.mark.parametrize("transpose", [True, False])
@pytest.mark.parametrize("d_out", [96, 128])
def test_kquant_fused_encode(cp, qt, transpose, d_out):
    """fused lift+encode == kquant_to_field -> (transpose) -> row packing -> encode (with PRG pad)"""
    from verinf_b200 import kquant_cuda as kq
    rng = np.random.default_rng(23)
    d_in, ell, k, n = 512, 1000, 2048, 8192
    raw = synth_blocks(rng, qt, d_out * d_in // 256)
    S = 1 << 12
    lifted = oracle.kquant_to_field(raw, qt, S).reshape(d_out, d_in)
    flat = (lifted.T if transpose else lifted).reshape(-1)
    rows = (flat.size + ell - 1) // ell
    msg = np.zeros(rows * ell, dtype=np.uint64)
    msg[:flat.size] = flat
    msg = msg.reshape(rows, ell)
    seed = bytes(range(7, 39))
    seed_t = torch.tensor(list(seed), dtype=torch.uint8, device="cuda")
    want_p, want_c = cp.encode_rows(dev(msg), k, n, master_seed=seed_t, row_offset=5)
    padded = np.zeros((rows, k), dtype=np.uint64)
    padded[:, :ell] = msg
    padded[:, ell:] = oracle.row_prg(seed, 5, rows, k - ell)
    _, oc = oracle.encode_rows(padded[:3], n)
    assert np.array_equal(host(want_c)[:3], oc)
    p, c = kq.kquant_encode_rows(torch.from_numpy(raw).cuda(), qt, S, d_out, d_in, ell=ell, k_deg=k, n_lig=n,
                                 transpose=transpose, master_seed=seed_t, row_offset=5, need_polys=True)
    assert torch.equal(c.view(torch.int64), want_c.view(torch.int64))
    assert torch.equal(p.view(torch.int64), want_p.view(torch.int64))
    p2, c2 = kq.kquant_encode_rows(torch.from_numpy(raw).cuda(), qt, S, d_out, d_in, ell=ell, k_deg=k, n_lig=n,
                                   transpose=transpose, first_row=7, n_rows=9, master_seed=seed_t, row_offset=12)
    assert p2 is None and torch.equal(c2.view(torch.int64), want_c[7:16].view(torch.int64))
    # scratch with room for one row chunk only: no staging area, the loader decodes from the super-blocks
    from verinf_b200._lib import LIB, check, ptr, stream_ptr
    small = torch.empty(((k + n) * 8,), dtype=torch.uint8, device="cuda")
    c3 = torch.empty((rows, n), dtype=torch.uint64, device="cuda")
    check(LIB.vi_kquant_encode_rows(ptr(torch.from_numpy(raw).cuda()), int(qt[1]), float(S), d_out, d_in, int(transpose),
                                    0, rows, ell, k, n, 1, ptr(seed_t), 5, None, ptr(c3), ptr(small), small.numel(),
                                    stream_ptr()))
    assert torch.equal(c3.view(torch.int64), want_c.view(torch.int64))


# ---------------------------------------------------------------- sumcheck ---
def _terms_from(g, name):
    terms = []
    for row in g[f"{name}_terms"]:
        vals = [int(v) for v in row]
        terms.append((vals[0], [v for v in vals[1:] if v >= 0]))
    return terms


@pytest.mark.parametrize("name", ["deg3_n6", "deg2_n4", "terms_n6", "mixed_n8", "single_n1"])
def test_sumcheck_golden(golden, name):
    from verinf_b200 import layergkr_gpu as lg
    g = golden.sumcheck_vectors
    tabs = g[f"{name}_tables"]
    coins = [int(c) for c in g[f"{name}_coins"]]
    dts = [dev(t) for t in tabs]
    terms = [(c, [dts[i] for i in idx]) for c, idx in _terms_from(g, name)]
    claim, polys, chals, mu = lg.prove_terms_gpu(terms, lambda i: coins[i])
    assert claim == int(g[f"{name}_claim"][0])
    assert [[y for _, y in rp] for rp in polys] == [[int(v) for v in row] for row in g[f"{name}_polys"]]
    assert [[x for x, _ in rp] for rp in polys] == [list(range(len(rp))) for rp in polys]
    assert chals == coins and mu == 0
    # python-list factors (the reference's calling convention) give the same transcript
    terms_l = [(c, [[int(v) for v in tabs[i]] for i in idx]) for c, idx in _terms_from(g, name)]
    claim2, polys2, _, _ = lg.prove_terms_gpu(terms_l, lambda i: coins[i])
    assert claim2 == claim and polys2 == polys


def _mask_fn(tape_vals):
    """mask(deg, mu) -> ascending coefficients of h with h(0) + h(1) = mu, drawing deg tape values
    (layergkr/sumcheck.py:73-92: MaskTape.take + mask_poly_coeffs)."""
    pos = [0]
    inv2 = pow(2, P - 2, P)

    def mask(deg, mu):
        u = tape_vals[pos[0]:pos[0] + deg]
        assert len(u) == deg, "mask tape exhausted"
        pos[0] += deg
        return [((mu - sum(u)) % P) * inv2 % P] + [x % P for x in u]
    return mask


@pytest.mark.parametrize("name", ["m_deg2_n4", "m_deg3_n6", "m_terms_n8"])
def test_sumcheck_masked_golden(golden, name):
    """Masked prover (layergkr/sumcheck.py:192-224, layergkr/gpu.py:395-406): the mask touches the
    scalar samples only; transcript, claim and carried mask equal the reference's CPython prover."""
    from verinf_b200 import layergkr_gpu as lg
    g = golden.sumcheck_masked_vectors
    tabs = g[f"{name}_tables"]
    coins = [int(c) for c in g[f"{name}_coins"]]
    tape = [int(v) for v in g[f"{name}_tape"]]
    mu0 = int(g[f"{name}_mu0"][0])
    dts = [dev(t) for t in tabs]
    terms = [(c, [dts[i] for i in idx]) for c, idx in _terms_from(g, name)]
    claim, polys, chals, mu = lg.prove_terms_gpu(terms, lambda i: coins[i], P, _mask_fn(tape), mu0)
    assert claim == int(g[f"{name}_claim"][0])
    assert [[y for _, y in rp] for rp in polys] == [[int(v) for v in row] for row in g[f"{name}_polys"]]
    assert chals == coins and mu == int(g[f"{name}_final_mask"][0])
    # the same proof with every round queued (challenges drawn before the first round), masks applied afterwards
    again = lg.prove_terms_gpu(terms, lambda i: coins[i], P, _mask_fn(tape), mu0, predraw=True)
    assert again == (claim, polys, chals, mu)


@pytest.mark.parametrize("logn,terms", [(12, [(1, [0, 1, 2])]), (16, [(1, [0, 1, 2])]), (13, [(3, [0, 1]), (P - 1, [2])]),
                                        (10, [(1, [0, 1, 2, 3])]), (15, [(1, [0, 0])]), (11, [(2, [1, 0, 2])])])
def test_sumcheck_vs_oracle(logn, terms):
    from verinf_b200 import layergkr_gpu as lg
    rng = np.random.default_rng(logn)
    ntab = 1 + max(max(f) for _, f in terms)
    tabs = rnd_field(rng, (ntab, 1 << logn))
    coins = [int(c) for c in rnd_field(rng, logn)]
    claim, samples, finals = oracle.sumcheck(tabs, terms, coins)
    prob = lg.SumcheckProblem(dev(tabs), terms)
    assert prob.claim() == claim
    r = None
    for rnd in range(logn):
        ys = prob.round(r)
        assert ys == [int(v) for v in samples[rnd][:len(ys)]], rnd
        r = coins[rnd]
    assert prob.round(r) is None
    assert prob.finals() == [int(v) for v in finals]
    prob2 = lg.SumcheckProblem(dev(tabs), terms)          # all rounds queued at once, coins known up front
    got = prob2.run(coins)
    assert got == [[int(v) for v in row[:len(got[0])]] for row in samples]
    assert prob2.finals() == [int(v) for v in finals]
    prob3 = lg.SumcheckProblem(dev(tabs), terms)          # g(1) filled on the host instead of by vi_sumcheck_complete
    rows = lg.samples_to_host(prob3.run_device(coins), prob3.deg)
    assert all(row[1] == 0 for row in rows[1:]) and lg.SumcheckProblem.complete_samples(rows, coins) == got


@pytest.mark.parametrize("logn,nt,nterms,predraw", [(9, 12, 20, False), (11, 30, 41, True), (7, 9, 3, True)])
def test_sumcheck_many_tables_and_terms_vs_oracle(logn, nt, nterms, predraw):
    """More tables / terms than one launch takes (a layer's gate batch, layergkr/relations.py:103-124): the terms
    are split into groups, mixed degrees are extended to the common sample count, samples are added."""
    from verinf_b200 import layergkr_gpu as lg
    rng = np.random.default_rng(100 * logn + nt)
    tabs = rnd_field(rng, (nt, 1 << logn))
    terms = [(int(rng.integers(1, 1 << 40)), [int(x) for x in rng.integers(0, nt, size=int(rng.integers(1, 5)))])
             for _ in range(nterms)]
    terms[0] = (P - 3, [0, 1, 2, 3])                      # at least one term of full degree
    coins = [int(c) for c in rnd_field(rng, logn)]
    claim, samples, _ = oracle.sumcheck(tabs, terms, coins)
    dts = [dev(t) for t in tabs]
    got = lg.prove_terms_gpu([(c, [dts[i] for i in idx]) for c, idx in terms], lambda i: coins[i], P, predraw=predraw)
    assert got[0] == claim and got[2] == coins
    assert [[y for _, y in rp] for rp in got[1]] == [[int(v) for v in row[:5]] for row in samples]


# ---------------------------------------------------------------- misc ops ---
def test_linear_algebra(cp):
    rng = np.random.default_rng(5)
    A, B = rnd_field(rng, (37, 65)), rnd_field(rng, (65, 41))
    C = host(cp.gl_matmul(dev(A), dev(B)))
    for (i, j) in ((0, 0), (36, 40), (17, 3)):
        assert int(C[i, j]) == sum(int(A[i, l]) * int(B[l, j]) for l in range(65)) % P
    # tile edges, the unaligned loader (odd n / odd k), more than one reduction period (k > 1024)
    for (m_, k_, n_) in ((64, 32, 32), (70, 2100, 45), (130, 1025, 64), (3, 1, 2), (64, 4096, 96), (33, 999, 34)):
        A2, B2 = rnd_field(rng, (m_, k_)), rnd_field(rng, (k_, n_))
        assert np.array_equal(host(cp.gl_matmul(dev(A2), dev(B2), force_simt=True)), oracle.gl_matmul(A2, B2)), (m_, k_, n_)
    # largest operands: every limb product and every accumulator at its bound
    A3 = np.full((64, 3072), P - 1, dtype=np.uint64)
    B3 = np.full((3072, 32), P - 1, dtype=np.uint64)
    assert np.array_equal(host(cp.gl_matmul(dev(A3), dev(B3), force_simt=True)), oracle.gl_matmul(A3, B3))
    A3[:] = np.uint64(0xFFFFFFFEFFFFFFFF)      # below p, both 32-bit limbs of a near their maximum
    B3[:] = np.uint64(0xFFFFEFFFFFFFFFFF)      # below p, the two 22-bit limbs of b all ones
    assert np.array_equal(host(cp.gl_matmul(dev(A3), dev(B3), force_simt=True)), oracle.gl_matmul(A3, B3))
    z = cp.gl_matmul(dev(A2[:, :0]), dev(B2[:0]))
    assert tuple(z.shape) == (33, 34) and not host(z).any()
    v = rnd_field(rng, 65)
    w = host(cp.gl_matvec(dev(A), dev(v)))
    assert [int(x) for x in w] == [sum(int(a) * int(b) for a, b in zip(A[i], v)) % P for i in range(37)]
    # CSR
    n_rows, n_cols = 9, 20
    row_ptr, col_idx, vals = [0], [], []
    for _ in range(n_rows):
        k = int(rng.integers(0, 6))
        col_idx += [int(c) for c in rng.integers(0, n_cols, size=k)]
        vals += [int(x) for x in rnd_field(rng, k)]
        row_ptr.append(len(col_idx))
    x = rnd_field(rng, n_cols)
    y = host(cp.gl_spmv(dev(vals), dev(col_idx), dev(row_ptr), dev(x), n_rows))
    for i in range(n_rows):
        s = sum(vals[p] * int(x[col_idx[p]]) for p in range(row_ptr[i], row_ptr[i + 1])) % P
        assert int(y[i]) == s
    seed = bytes(range(32))
    seed_t = torch.tensor(list(seed), dtype=torch.uint8, device="cuda")
    lab = torch.tensor(list(b"lin"), dtype=torch.uint8, device="cuda")
    y2 = host(cp.gl_spmv_challenged(dev(vals), dev(col_idx), dev(row_ptr), seed_t, lab, n_rows))
    for i in range(n_rows):
        s = sum(vals[p] * oracle.challenge(seed, col_idx[p], b"lin") for p in range(row_ptr[i], row_ptr[i + 1])) % P
        assert int(y2[i]) == s


def test_lookup_multiplicities(cp):
    x = dev([0, 3, 3, 7, 9, 100, 3])
    table = dev(list(range(8)))
    m = host(cp.lookup_multiplicities(x, table))
    assert [int(v) for v in m] == [1, 0, 0, 3, 0, 0, 0, 1]
    acc = torch.zeros(8, dtype=torch.uint64, device="cuda")
    cp.lookup_multiplicities_into(x, table, acc)
    cp.lookup_multiplicities_into(x, table, acc)
    assert [int(v) for v in host(acc)] == [2, 0, 0, 6, 0, 0, 0, 2]
    t2 = dev([5, 9, 100, 3])
    acc2 = torch.zeros(4, dtype=torch.uint64, device="cuda")
    cp.lookup_multiplicities_into(x, t2, acc2)
    assert [int(v) for v in host(acc2)] == [0, 1, 1, 3]


def test_interp_bands(cp):
    seed = bytes(range(32))
    seed_t = torch.tensor(list(seed), dtype=torch.uint8, device="cuda")
    lab = torch.tensor(list(b"lin"), dtype=torch.uint8, device="cuda")
    ch = lambda c: oracle.challenge(seed, c, b"lin")   # noqa: E731
    n = 24
    out = torch.zeros(n + 4, dtype=torch.uint64, device="cuda")
    # causal_id: base, m, h, coef
    cp.interp_band_causal_id(out, 2, 5, n, 1000, 4, 3, 11, seed_t, lab)
    got = host(out)
    for s in range(n):
        f = 5 + s
        b, j = divmod(f, 4)
        iq, hh = divmod(b, 3)
        want = 0 if j > iq else 11 * ch(1000 + 3 * iq * (iq + 1) // 2 + hh * (iq + 1) + j) % P
        assert int(got[2 + s]) == want
    assert not got[:2].any() and not got[2 + n:].any()
    # descriptor band, const coef, PRF challenges, fan 2
    desc = [0] * 24
    desc[0] = 2; desc[1] = 1; desc[2] = 5; desc[5] = 70; desc[6] = 10; desc[7] = 1
    desc[10] = 2; desc[11] = 100; desc[12] = 0; desc[13] = 9
    out2 = torch.zeros(n, dtype=torch.uint64, device="cuda")
    z = torch.zeros(1, dtype=torch.uint64, device="cuda")
    cp.interp_band(out2, 0, 3, n, dev(desc), z, z, z, seed_t, lab)
    got2 = host(out2)
    for s in range(n):
        hi, lo = divmod(3 + s, 5)
        cid = 70 + hi * 10 + lo
        assert int(got2[s]) == 9 * ((ch(cid) + ch(cid + 100)) % P) % P


# ---------------------------------------------------------------- sharded column hash ---
@pytest.mark.parametrize("m,n,world", [(1024, 300, 2), (4096, 64, 8), (1000, 77, 3), (700, 40, 4), (129, 9, 2)])
def test_sharded_hash_emulated_ranks(cp, m, n, world):
    """sub-tree chaining values of every rank's aligned blocks, folded, equal the whole-matrix digests"""
    from verinf_b200 import distributed as D
    rng = np.random.default_rng(m + n)
    a = rnd_field(rng, (m, n))
    t = dev(a)
    be = D.CudaBackend(0, 0)
    cvs, levels = [], []
    for r0, r1 in D.split_rows(m, world):
        for b0, cnt, lvl in D.aligned_blocks(r0, r1):
            cv = be.hash_subtree(t[b0:b0 + cnt], b0 // 128, lvl)
            assert np.array_equal(cv.cpu().numpy(), oracle.hash_subtree(a[b0:b0 + cnt], b0 // 128))
            cvs.append(cv)
            levels.append(lvl)
    got = be.merge(torch.stack(cvs).contiguous(), levels)
    assert np.array_equal(got.cpu().numpy(), oracle.hash_columns(a))


def test_commit_rows_sharded_single_process(cp):
    from verinf_b200 import distributed as D
    rng = np.random.default_rng(8)
    msg = dev(rnd_field(rng, (600, 100)))
    root, levels, codes = D.commit_rows_sharded(msg, 600, D.CudaBackend(128, 512))
    want_root, _, want_codes = cp.commit_rows(msg, 128, 512)
    assert torch.equal(root, want_root) and torch.equal(codes.view(torch.int64), want_codes.view(torch.int64))


def test_more_rows_than_a_grid_dimension(cp):
    """70000 rows in one call: the reference's batched kernels stop at 65535 rows (one block-row per
    message, layergkr/gpu.py:33-35); here rows are tiled, so there is no such cap."""
    rng = np.random.default_rng(65536)
    m = 70000
    a = rnd_field(rng, (m, 64))
    x = dev(a)
    cp.ntt_forward_batched(x)
    got = host(x)
    idx = [0, 1, 65534, 65535, 65536, m - 1]
    assert np.array_equal(got[idx], oracle.ntt_batched(a[idx]))
    msg = rnd_field(rng, (m, 6))
    _, codes = cp.encode_rows(dev(msg), 8, 32, need_polys=False)
    padded = np.zeros((len(idx), 8), dtype=np.uint64)
    padded[:, :6] = msg[idx]
    assert np.array_equal(host(codes)[idx], oracle.encode_rows(padded, 32, want_polys=False)[1])
    leaves = cp.hash_columns_streamed(codes)
    assert np.array_equal(leaves.cpu().numpy(), oracle.hash_columns(host(codes)))


@pytest.mark.parametrize("m,k,n", [(1, 1000, 70), (1, 4096, 16384), (2, 300, 33), (3, 129, 1), (4, 2048, 100), (1, 7, 5),
                                   (200, 513, 1), (1, 1, 1)])
def test_matmul_thin_shapes(cp, m, k, n):
    """row combinations (m <= 4) and single-column products take their own kernels"""
    rng = np.random.default_rng(m * 1000 + k + n)
    A, B = rnd_field(rng, (m, k)), rnd_field(rng, (k, n))
    assert np.array_equal(host(cp.gl_matmul(dev(A), dev(B))), oracle.gl_matmul(A, B))
    A[:] = np.uint64(0xFFFFFFFEFFFFFFFF)
    B[:] = np.uint64(P - 1)
    assert np.array_equal(host(cp.gl_matmul(dev(A), dev(B))), oracle.gl_matmul(A, B))


def _matmul_tc(A, B):
    from verinf_b200._lib import LIB, check, ptr, stream_ptr
    m, k = A.shape
    n = B.shape[1]
    nb = LIB.vi_gl_matmul_tc_scratch_bytes(m, k, n)
    sc = torch.empty(max(nb, 16), dtype=torch.uint8, device="cuda")
    out = torch.empty((m, n), dtype=torch.uint64, device="cuda")
    a_d, b_d = dev(A), dev(B)
    check(LIB.vi_gl_matmul_tc(ptr(a_d), ptr(b_d), ptr(out), m, k, n, ptr(sc), nb, stream_ptr()))
    return host(out)


@pytest.mark.parametrize("m,k,n", [(64, 32, 32), (1, 1, 1), (3, 5, 2), (70, 2100, 45), (130, 4096, 64), (65, 4097, 33),
                                   (16, 9000, 40), (200, 300, 500)])
def test_matmul_tensor_cores_vs_oracle(cp, m, k, n):
    """byte-plane product on the integer tensor cores: ragged tiles, several 4096-term chunks"""
    rng = np.random.default_rng(m * 7 + k + n)
    A, B = rnd_field(rng, (m, k)), rnd_field(rng, (k, n))
    assert np.array_equal(_matmul_tc(A, B), oracle.gl_matmul(A, B))


def _matmul_umma(A, B):
    """vi_gl_matmul_umma through the C ABI, with its device status word checked."""
    from verinf_b200._lib import LIB, check, ptr, stream_ptr
    m, k = A.shape
    n = B.shape[1]
    nb = LIB.vi_gl_matmul_umma_scratch_bytes(m, k, n)
    sc = torch.empty(max(nb, 256), dtype=torch.uint8, device="cuda")
    st = torch.full((1,), 77, dtype=torch.int32, device="cuda")
    out = torch.empty((m, n), dtype=torch.uint64, device="cuda")
    a_d, b_d = dev(A), dev(B)
    check(LIB.vi_gl_matmul_umma(ptr(a_d), ptr(b_d), ptr(out), m, k, n, ptr(sc), nb, ptr(st), stream_ptr()))
    torch.cuda.synchronize()
    assert int(st.item()) == 0, "a bounded wait of the tcgen05 kernel expired"
    return host(out)


@pytest.mark.parametrize("m,k,n", [(128, 64, 32), (1, 1, 1), (3, 5, 2), (70, 2100, 45), (130, 4096, 64), (65, 4097, 33),
                                   (16, 9000, 40), (200, 300, 500), (257, 8193, 31)])
def test_matmul_tcgen05_vs_oracle(cp, m, k, n):
    """byte-plane product with tensor-memory accumulators (tcgen05.mma kind::i8): ragged tiles, k not a
    multiple of the 64-byte stage, several 4096-term chunks (accumulators restarted per chunk)"""
    rng = np.random.default_rng(m * 11 + k + n)
    A, B = rnd_field(rng, (m, k)), rnd_field(rng, (k, n))
    assert np.array_equal(_matmul_umma(A, B), oracle.gl_matmul(A, B))


def test_matmul_tcgen05_extreme_operands_and_dispatch(cp):
    # every byte 0xff where the field allows it: all 15 plane sums reach their bound within a chunk
    A = np.full((128, 8192), 0xFFFFFFFEFFFFFFFF, dtype=np.uint64)
    B = np.full((8192, 32), 0xFFFFFFFEFFFFFFFF, dtype=np.uint64)
    assert np.array_equal(_matmul_umma(A, B), oracle.gl_matmul(A, B))
    A[:] = np.uint64(P - 1)
    assert np.array_equal(_matmul_umma(A, B), oracle.gl_matmul(A, B))
    # the Python entry point takes this path from 2^26 multiply-adds; all three kernels agree
    rng = np.random.default_rng(2)
    A, B = rnd_field(rng, (520, 1030)), rnd_field(rng, (1030, 260))
    got = cp.gl_matmul(dev(A), dev(B))
    assert torch.equal(got.view(torch.int64), cp.gl_matmul(dev(A), dev(B), path="umma").view(torch.int64))
    assert torch.equal(got.view(torch.int64), cp.gl_matmul(dev(A), dev(B), path="mma").view(torch.int64))
    assert torch.equal(got.view(torch.int64), cp.gl_matmul(dev(A), dev(B), path="simt").view(torch.int64))
    cp.check_async_errors()
    assert np.array_equal(host(got)[:7], oracle.gl_matmul(A[:7], B))


def test_matmul_tensor_cores_extreme_operands(cp):
    # every byte 0xff where the field allows it: all 15 plane sums reach their bound within a chunk
    A = np.full((64, 8192), 0xFFFFFFFEFFFFFFFF, dtype=np.uint64)
    B = np.full((8192, 32), 0xFFFFFFFEFFFFFFFF, dtype=np.uint64)
    assert np.array_equal(_matmul_tc(A, B), oracle.gl_matmul(A, B))
    A[:] = np.uint64(P - 1)
    assert np.array_equal(_matmul_tc(A, B), oracle.gl_matmul(A, B))
    # the Python entry point takes the tensor-core path for large products and the scalar one otherwise
    rng = np.random.default_rng(1)
    A, B = rnd_field(rng, (256, 512)), rnd_field(rng, (512, 128))
    got = cp.gl_matmul(dev(A), dev(B))
    assert np.array_equal(host(got), oracle.gl_matmul(A, B))
    assert torch.equal(got.view(torch.int64), cp.gl_matmul(dev(A), dev(B), force_simt=True).view(torch.int64))


# ---------------------------------------------------------------- openings ----
@pytest.mark.parametrize("n", [1, 2, 5, 8, 13])
def test_merkle_paths_golden(cp, golden, n):
    from verinf_b200 import commit
    g = golden.merkle_path_vectors
    leaves = torch.from_numpy(g[f"n{n}_leaves"].copy()).cuda()
    root, levels = cp.merkle_build_blake3(leaves)
    assert root.cpu().numpy().tobytes() == g[f"n{n}_root"].tobytes()
    upper = torch.empty((1, 32), dtype=torch.uint8, device="cuda") if n == 1 else torch.cat(levels[1:]).contiguous()
    sib, sides = commit.merkle_paths(leaves, upper, list(range(n)))
    assert np.array_equal(sib.cpu().numpy(), g[f"n{n}_siblings"])
    assert np.array_equal(sides.cpu().numpy(), g[f"n{n}_sides"])


@pytest.mark.parametrize("n", [1000, 4097, 65536])
def test_merkle_paths_vs_oracle(cp, n):
    from verinf_b200 import commit
    rng = np.random.default_rng(n)
    leaves_h = rng.integers(0, 256, size=(n, 32), dtype=np.uint8)
    leaves = torch.from_numpy(leaves_h).cuda()
    root, levels = cp.merkle_build_blake3(leaves)
    upper = torch.cat(levels[1:]).contiguous()
    q = sorted(set([0, 1, n - 1, n - 2, n // 2] + [int(v) for v in rng.integers(0, n, size=40)]))
    sib, sides = commit.merkle_paths(leaves, upper, q)
    want_levels = oracle.merkle_levels(leaves_h)
    got = commit.paths_as_reference(sib, sides)
    root_b = root.cpu().numpy().tobytes()
    for t, j in enumerate(q):
        assert got[t] == oracle.merkle_path(want_levels, j)
        assert oracle.merkle_verify(leaves_h[j].tobytes(), got[t], root_b)
    with pytest.raises(RuntimeError):
        commit.merkle_paths(leaves, upper, [n])


def test_open_columns_and_committer_open(cp):
    from verinf_b200 import commit
    rng = np.random.default_rng(8)
    rows, ell, k, n = 300, 48, 64, 256
    msg = rnd_field(rng, (rows, ell))
    seed_t = torch.arange(32, dtype=torch.uint8, device="cuda")
    com = commit.RowCommitter(rows, ell, k, n, master_seed=seed_t)
    root = com.commit(dev(msg), row_offset=3).cpu().numpy().tobytes()
    q = [0, 255, 17, 17, 128, 3]
    cols, sib, sides = com.open(q)
    codes = host(com.codes)
    assert np.array_equal(host(cols), codes[:, q].T)
    leaves = oracle.hash_columns(codes)
    for t, j in enumerate(q):
        path = commit.paths_as_reference(sib, sides)[t]
        assert oracle.merkle_verify(leaves[j].tobytes(), path, root)
        # the opened column hashes to the leaf the path authenticates (core.py:1086 check)
        assert oracle.blake3(host(cols)[t].tobytes()) == leaves[j].tobytes()
    with pytest.raises(RuntimeError):
        com.open([256])
    assert tuple(commit.open_columns(com.codes, []).shape) == (0, rows)


@pytest.mark.parametrize("chunks", [[600], [100, 1, 127, 300, 72], [128, 128, 128, 216], [1] * 3 + [597]])
def test_stream_committer_equals_one_shot(cp, chunks):
    from verinf_b200 import commit
    rng = np.random.default_rng(5)
    total, ell, k, n = sum(chunks), 100, 128, 512
    msg = dev(rnd_field(rng, (total, ell)))
    seed_t = torch.arange(32, dtype=torch.uint8, device="cuda")
    want_root, want_levels, want_codes = cp.commit_rows(msg, k, n, master_seed=seed_t, row_offset=77)
    q = [5, 500, 0, 511]
    sc = commit.StreamCommitter(total, ell, k, n, master_seed=seed_t, row_offset=77, open_cols=q, max_chunk_rows=256)
    r0 = 0
    for c in chunks:
        sc.update(msg[r0:r0 + c])
        r0 += c
    root = sc.finalize()
    assert torch.equal(root, want_root)
    assert torch.equal(sc.opened.view(torch.int64), want_codes.view(torch.int64)[:, q].T)
    sib, sides = sc.paths()
    levels = oracle.merkle_levels(want_levels[0].cpu().numpy())
    assert commit.paths_as_reference(sib, sides) == [oracle.merkle_path(levels, j) for j in q]


# ---------------------------------------------------------------- folds -------
@pytest.mark.parametrize("name", ["small", "indexed"])
def test_fold_golden(cp, golden, name):
    from verinf_b200 import fold
    g = golden.fold_vectors
    A, B, w = dev(g[f"{name}_A"]), dev(g[f"{name}_B"]), dev(g[f"{name}_w"])
    ia, ib = torch.from_numpy(g[f"{name}_ia"]).cuda(), torch.from_numpy(g[f"{name}_ib"]).cuda()
    n_eval = fold.eval_size(A.size(1))
    assert n_eval == g[f"{name}_eval_ones"].size
    EA, EB = fold.ntt_forward_padded(A, n_eval), fold.ntt_forward_padded(B, n_eval)
    assert np.array_equal(host(fold.product_colsum(EA, EB, w, ia, ib)), g[f"{name}_eval_weighted"])
    assert np.array_equal(host(fold.product_colsum(EA, EB, None, ia, ib)), g[f"{name}_eval_ones"])
    acc = fold.product_colsum(EA, EB, w, ia, ib)
    cp.ntt_inverse(acc)
    k2 = g[f"{name}_coef"].size
    assert np.array_equal(host(acc)[:k2], g[f"{name}_coef"]) and not host(acc)[k2:].any()
    if name == "small":
        assert np.array_equal(host(fold.fold_products_eval(A, B, w)), g[f"{name}_eval_weighted"])


@pytest.mark.parametrize("m,k", [(1, 2), (7, 64), (33, 512), (40, 1024), (9, 4096), (300, 2048), (5, 16384)])
def test_fold_vs_oracle_and_reference_composition(cp, m, k):
    from verinf_b200 import fold
    rng = np.random.default_rng(m * 31 + k)
    A, B, w = rnd_field(rng, (m, k)), rnd_field(rng, (m, k)), rnd_field(rng, m)
    n_eval = fold.eval_size(k)
    got = fold.fold_products_eval(dev(A), dev(B), dev(w))
    assert np.array_equal(host(got), oracle.fold_products_eval(A, B, n_eval, w))
    ones = fold.fold_products_eval(dev(A), dev(B))
    assert np.array_equal(host(ones), oracle.fold_products_eval(A, B, n_eval))
    # the reference's own sequence on the drop-in primitives (prover/core.py:1900-1911)
    a_pad = torch.zeros((m, n_eval), dtype=torch.uint64, device="cuda"); a_pad[:, :k] = dev(A)
    b_pad = torch.zeros((m, n_eval), dtype=torch.uint64, device="cuda"); b_pad[:, :k] = dev(B)
    assert torch.equal(fold.ntt_forward_padded(dev(A), n_eval).view(torch.int64),
                       (cp.ntt_forward_batched(a_pad), a_pad)[1].view(torch.int64))
    cp.ntt_forward_batched(b_pad)
    prod = cp.gl_mul(a_pad, b_pad)
    ref = cp.gl_matvec(prod.view(torch.int64).T.contiguous().view(torch.uint64),
                       torch.ones(m, dtype=torch.int64, device="cuda").view(torch.uint64))
    assert torch.equal(ref.view(torch.int64), ones.view(torch.int64))
    # accumulation into an existing buffer and linearity of the inverse transform
    acc = ones.clone()
    fold.fold_products_eval(dev(A), dev(B), dev(w), out=acc)
    assert np.array_equal(host(acc), host(cp.gl_add(ones, got)))
    if k <= 1024:
        cp.ntt_inverse(ones)
        pm = cp.poly_mul_batched(dev(A), dev(B))
        s = host(cp.gl_matvec(pm.view(torch.int64).T.contiguous().view(torch.uint64),
                              torch.ones(m, dtype=torch.int64, device="cuda").view(torch.uint64)))
        assert np.array_equal(host(ones)[:2 * k - 1], s)


def test_fold_indexed_rows_and_edges(cp):
    from verinf_b200 import fold
    rng = np.random.default_rng(4)
    rows, k, T = 50, 256, 700
    A, B, w = rnd_field(rng, (rows, k)), rnd_field(rng, (rows + 3, k)), rnd_field(rng, T)
    ia, ib = rng.integers(0, rows, size=T), rng.integers(0, rows + 3, size=T)
    n_eval = fold.eval_size(k)
    EA, EB = fold.ntt_forward_padded(dev(A), n_eval), fold.ntt_forward_padded(dev(B), n_eval)
    got = fold.product_colsum(EA, EB, dev(w), torch.from_numpy(ia).cuda(), torch.from_numpy(ib).cuda())
    assert np.array_equal(host(got), oracle.fold_products_eval(A, B, n_eval, w, ia, ib))
    # largest operands: every product and the carry limb at their bounds
    big = torch.full((600, 512), -(1 << 32), dtype=torch.int64, device="cuda").view(torch.uint64)   # p - 1
    s = fold.product_colsum(big, big)
    assert host(s).tolist() == [600 % P] * 512
    e = torch.empty((0, 512), dtype=torch.uint64, device="cuda")
    assert not host(fold.product_colsum(e, e)).any()
    with pytest.raises(RuntimeError):
        fold.product_colsum(EA, EB)                         # row counts differ and no indices
    with pytest.raises(RuntimeError):
        fold.product_colsum(EA, EB, None, torch.tensor([rows], device="cuda"), torch.tensor([0], device="cuda"))
    with pytest.raises(RuntimeError):
        fold.ntt_forward_padded(dev(A), 128)                # rows longer than the transform


@pytest.mark.parametrize("rows,slices", [(600, 16), (2100, 16), (4096, 16), (1024, 3), (129, 1), (100, 4)])
def test_commit_host_equals_device_commit(cp, rows, slices):
    """pinned-host commit (sliced copies overlapped with the encode, column hash streamed per slice)
    gives the root of the one-shot device commit"""
    from verinf_b200 import commit
    rng = np.random.default_rng(rows)
    ell, k, n = 48, 64, 256
    msg = rnd_field(rng, (rows, ell))
    seed_t = torch.arange(32, dtype=torch.uint8, device="cuda")
    com = commit.RowCommitter(rows, ell, k, n, master_seed=seed_t, h2d_slices=slices)
    want = com.commit(dev(msg), row_offset=9).cpu().numpy().tobytes()
    pinned = torch.from_numpy(msg.view(np.int64)).view(torch.uint64).pin_memory()
    assert com.commit_host(pinned, row_offset=9) == want
    assert com.commit_host(pinned, row_offset=9) == want          # buffers are reused
    padded = np.zeros((rows, k), dtype=np.uint64)
    padded[:, :ell] = msg
    padded[:, ell:] = oracle.row_prg(bytes(range(32)), 9, rows, k - ell)
    assert oracle.commit_rows(padded, n) == want


# ---------------------------------------------------------------- layergkr helpers ----
def test_layergkr_helper_mirrors(cp, golden):
    """the helpers of layergkr/gpu.py around the hot path: same values as their definitions"""
    from types import SimpleNamespace
    from verinf_b200 import layergkr_gpu as lg
    g = golden.encode_vectors
    cfg = SimpleNamespace(ELL=16, K_DEG=32, N_LIG=128)
    msg = g["msg_16_32_128"]
    rows = [[int(v) for v in r] for r in msg]
    want = g["code_16_32_128"]
    assert lg.available()
    assert np.array_equal(np.array(lg.encode_batch(cfg, rows), dtype=np.uint64), want)
    codes = lg.encode_batch_t(cfg, rows)
    assert np.array_equal(host(codes), want)
    rng = np.random.default_rng(2)
    coeffs = [int(v) for v in rnd_field(rng, msg.shape[0])]
    comb = [sum(c * int(want[i, j]) for i, c in enumerate(coeffs)) % P for j in range(128)]
    assert [int(v) for v in host(lg.combine_t(cfg, codes, coeffs))[0]] == comb
    assert lg.linear_combination(cfg, [[int(v) for v in r] for r in want], coeffs) == comb
    assert lg.column(codes, 77) == [int(v) for v in want[:, 77]]
    root, levels = lg.hash_and_tree(cfg, codes)
    assert root == g["root_16_32_128"].tobytes()
    assert b"".join(b"".join(l) for l in lg.levels_to_host(levels)) == g["tree_16_32_128"].tobytes()
    for n in (1, 7, 1024, 1025, 100003):
        v = rnd_field(rng, n)
        assert int(host(lg.gl_sum(dev(v)))[0]) == sum(int(x) for x in v) % P
    f = rnd_field(rng, 4096)
    r = int(rnd_field(rng, 1)[0])
    got = host(lg.fold_t(dev(f), dev(np.array([r], dtype=np.uint64))))
    assert [int(x) for x in got] == [(int(a) + r * (int(b) - int(a))) % P for a, b in zip(f[:2048], f[2048:])]


def test_release_tables_then_reuse(cp):
    """tables are rebuilt after vi_release_tables: same transform before and after"""
    from verinf_b200._lib import LIB, check
    rng = np.random.default_rng(3)
    a = rnd_field(rng, (3, 4096))
    x = dev(a)
    cp.ntt_forward_batched(x)
    torch.cuda.synchronize()
    check(LIB.vi_release_tables())
    y = dev(a)
    cp.ntt_forward_batched(y)
    assert torch.equal(x.view(torch.int64), y.view(torch.int64))
    _, c = cp.encode_rows(dev(a[:, :1000]), 4096, 16384)
    assert np.array_equal(host(c)[0], oracle.encode_rows(np.concatenate([a[:1, :1000], np.zeros((1, 3096), np.uint64)], 1), 16384)[1][0])
