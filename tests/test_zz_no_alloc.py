"""GPU: the allocation-free column hash (vi_hash_columns_noalloc) against the regular entry
point (vi_hash_columns), through the C ABI, on two calls in a row.

Who needs it: a host that cannot call cudaMalloc when it wants a column hash - a prover that
has given all free HBM to its witness and codeword buffers, or code that runs under a fixed
memory budget - so the state the regular entry point takes as caller scratch sits in a fixed
8 MiB device array inside the library.  Both calls below share that array; the second one must
not be disturbed by what the first one left in it.  Bit-exact comparison (integer work)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _digests(lib, mat, noalloc):
    m, n = mat.shape
    out = torch.zeros((n, 32), dtype=torch.uint8, device="cuda")
    if noalloc:
        lib.check(lib.LIB.vi_hash_columns_noalloc(mat.data_ptr(), m, n, out.data_ptr(), lib.stream_ptr()))
    else:
        nb = lib.LIB.vi_hash_columns_scratch_bytes(m, n)
        scratch = torch.empty(max(nb, 1), dtype=torch.uint8, device="cuda")
        lib.check(lib.LIB.vi_hash_columns(mat.data_ptr(), m, n, out.data_ptr(), scratch.data_ptr(), nb,
                                          lib.stream_ptr()))
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_noalloc_matches_regular_entry_point_twice():
    from verinf_b200 import _lib as lib
    rng = np.random.default_rng(2024)
    shapes = [(1000, 4096), (300, 777)]          # second call: fewer levels, other width, stale state behind it
    for m, n in shapes:
        a = rng.integers(0, (1 << 64) - (1 << 32) + 1, size=(m, n), dtype=np.uint64)
        mat = torch.from_numpy(a.view(np.int64)).cuda().view(torch.uint64)
        want = _digests(lib, mat, noalloc=False)
        got = _digests(lib, mat, noalloc=True)
        assert np.array_equal(got, want), (m, n)
    # single-chunk input (no state at all) and the size limit
    small = torch.arange(64 * 10, dtype=torch.int64, device="cuda").view(torch.uint64).reshape(64, 10)
    assert np.array_equal(_digests(lib, small, True), _digests(lib, small, False))
    limit = lib.LIB.vi_hash_columns_noalloc_max_state_bytes()
    assert limit == 8 << 20
    cols = 1 << 16
    assert lib.LIB.vi_hash_stream_state_bytes(cols, 1024) <= limit
    big = torch.zeros((2048, cols), dtype=torch.uint64, device="cuda")      # needs 5 levels x 2 MiB > 8 MiB
    out = torch.empty((cols, 32), dtype=torch.uint8, device="cuda")
    rc = lib.LIB.vi_hash_columns_noalloc(big.data_ptr(), 2048, cols, out.data_ptr(), lib.stream_ptr())
    assert rc == 4 and b"built-in buffer" in lib.LIB.vi_last_error()      # VI_ERR_LIMIT
