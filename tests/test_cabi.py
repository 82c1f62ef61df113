"""CPU: the C-ABI library loads, exports every symbol the header declares, and its host-side
argument validation and size helpers behave (no kernel is launched: there is no GPU here)."""
import ctypes as C
import re
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from verinf_b200 import _lib
    return _lib


def test_exports_every_declared_symbol(lib):
    hdr = (ROOT / "include" / "verinf_b200.h").read_text()
    declared = set(re.findall(r"\b(vi_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    raw = C.CDLL(str(lib.SO_PATH))
    for name in sorted(declared):
        assert hasattr(raw, name), f"{name} declared in the header but not exported"
    assert declared == set(lib.SIGNATURES), "ctypes signature table and header disagree"


def test_size_helpers(lib):
    L = lib.LIB
    assert L.vi_merkle_upper_nodes(1) == 0
    assert L.vi_merkle_upper_nodes(2) == 1
    assert L.vi_merkle_upper_nodes(5) == 3 + 2 + 1
    assert L.vi_merkle_upper_nodes(4096) == 4095
    assert L.vi_ntt_scratch_bytes(10, 1024) == 0
    assert L.vi_ntt_scratch_bytes(1, 1 << 16) == (1 << 16) * 8
    assert L.vi_ntt_scratch_bytes(1, 1 << 24) == (1 << 24) * 8
    assert L.vi_ntt_scratch_bytes(10 ** 6, 1 << 16) % ((1 << 16) * 8) == 0
    assert L.vi_encode_scratch_bytes(1, 1 << 10, 1 << 12) == ((1 << 10) + (1 << 12)) * 8
    assert L.vi_encode_scratch_bytes(0, 8, 32) == 0
    assert L.vi_hash_stream_state_bytes(100, 64) == 2 * 32 * 100          # one chunk: levels 0..1
    assert L.vi_hash_stream_state_bytes(100, 4096) == 6 * 32 * 100        # 32 chunks: levels 0..5
    assert L.vi_hash_stream_state_bytes(100, 4097) == 7 * 32 * 100
    assert L.vi_hash_columns_scratch_bytes(4096, 200000) == L.vi_hash_stream_state_bytes(200000, 4096)
    assert L.vi_hash_columns_scratch_bytes(4096, 100) > L.vi_hash_stream_state_bytes(100, 4096)   # row segments
    assert L.vi_hash_columns_scratch_bytes(100, 100) == L.vi_hash_stream_state_bytes(100, 100)
    assert L.vi_sumcheck_scratch_bytes() > 0
    assert L.vi_profile_num_tags() >= 9
    assert L.vi_profile_tag_name(0) == b"encode_pass1"


def _err(lib):
    return lib.LIB.vi_last_error().decode()


def test_argument_validation_without_gpu(lib):
    L = lib.LIB
    buf = (C.c_uint64 * 64)()
    p = C.cast(buf, C.c_void_p)
    assert L.vi_ntt_batched(p, 1, 12, 0, None, 0, None) != 0 and "power of 2" in _err(lib)
    assert L.vi_ntt_batched(p, 1, 1, 0, None, 0, None) != 0
    assert L.vi_ntt_batched(p, -1, 16, 0, None, 0, None) != 0
    assert L.vi_ntt_batched(p, 1, 1 << 31, 0, None, 0, None) != 0 and "exceeds" in _err(lib)
    assert L.vi_ntt_batched(p, 1, 1 << 25, 0, None, 0, None) != 0 and "scratch" in _err(lib)   # three passes: 2*n*8 bytes
    assert L.vi_ntt_batched(p, 0, 16, 0, None, 0, None) == 0                  # empty batch is fine
    assert L.vi_encode_rows(p, 1, 9, 8, 32, 0, None, 0, p, p, p, 1 << 20, None) != 0 and "ELL" in _err(lib)
    assert L.vi_encode_rows(p, 1, 8, 12, 48, 0, None, 0, p, p, p, 1 << 20, None) != 0
    assert L.vi_encode_rows(p, 1, 8, 8, 4, 0, None, 0, p, p, p, 1 << 20, None) != 0
    assert L.vi_encode_rows(p, 1, 4, 8, 32, 1, None, 0, p, p, p, 1 << 20, None) != 0 and "seed" in _err(lib)
    assert L.vi_encode_rows(p, 1, 8, 8, 32, 0, None, 0, p, p, None, 0, None) != 0 and "scratch" in _err(lib)
    assert L.vi_encode_rows(p, 0, 8, 8, 32, 0, None, 0, None, None, None, 0, None) == 0
    assert L.vi_gl_binary(7, p, p, p, 4, None) != 0
    assert L.vi_gl_binary(0, p, p, p, 0, None) == 0
    assert L.vi_kquant_to_field(p, 1, 3, 4096.0, p, None) != 0 and "qtype" in _err(lib)
    assert L.vi_hash_stream_update(p, 8, 256, 100, p, 128, p, None) != 0 and "multiple of 128" in _err(lib)
    assert L.vi_hash_stream_update(p, 8, 256, 0, p, 100, p, None) != 0 and "partial" in _err(lib)
    assert L.vi_hash_stream_update(p, 8, 256, 128, p, 256, p, None) != 0
    assert L.vi_hash_columns(p, 4096, 200000, p, None, 0, None) != 0 and "scratch" in _err(lib)
    assert L.vi_challenge(p, p, 9, None, 4, p, None) != 0 and "label" in _err(lib)
    assert L.vi_ntt_forward_padded(p, 1, 9, p, 8, None, 0, None) != 0 and "do not fit" in _err(lib)
    assert L.vi_ntt_forward_padded(p, 1, 8, p, 12, None, 0, None) != 0 and "power of 2" in _err(lib)
    assert L.vi_ntt_forward_padded(p, 0, 8, p, 16, None, 0, None) == 0
    assert L.vi_ntt_forward_padded(p, 1, 8, p, 1 << 12, None, 0, None) != 0          # aliasing / scratch
    assert L.vi_product_colsum(p, p, 16, None, None, None, 4, p, 0, None, 0, None) != 0 and "scratch" in _err(lib)
    assert L.vi_product_colsum(p, p, 0, None, None, None, 4, p, 0, None, 0, None) == 0
    assert L.vi_product_colsum_scratch_bytes(4, 16) == 16 * 8 and L.vi_product_colsum_scratch_bytes(0, 16) == 0
    assert L.vi_product_colsum_scratch_bytes(4096, 32768) == 5 * 32768 * 8
    assert L.vi_gl_matmul_tc(p, p, p, 4, 4, 4, None, 0, None) != 0 and "alias" in _err(lib)
    buf2 = (C.c_uint64 * 64)()
    assert L.vi_gl_matmul_tc(p, p, C.cast(buf2, C.c_void_p), 4, 4, 4, None, 0, None) != 0 and "scratch" in _err(lib)
    assert L.vi_gl_matmul_tc_scratch_bytes(1, 1, 1) == 8 * (64 + 32) * 64
    assert L.vi_gl_matmul_tc_scratch_bytes(1000, 4096, 11008) == 8 * (1024 + 11008) * 4096
    assert L.vi_gl_matmul_tc(p, p, p, 0, 4, 4, None, 0, None) == 0
    assert L.vi_open_columns(p, 4, 8, p, 2, p, 3, 0, None) != 0 and "stride" in _err(lib)
    assert L.vi_open_columns(p, -1, 8, p, 2, p, 3, 0, None) != 0
    assert L.vi_open_columns(p, 0, 8, p, 2, p, 3, 0, None) == 0
    assert L.vi_merkle_paths(p, 0, p, p, 1, p, p, None) != 0
    assert L.vi_merkle_paths(p, 1, p, p, 5, p, p, None) == 0                  # a single leaf has an empty path
    assert [L.vi_merkle_depth(n) for n in (1, 2, 3, 5, 8, 9, 4096)] == [0, 1, 2, 3, 3, 4, 12]
    coefs = (C.c_uint64 * 1)(1)
    nfac = (C.c_int32 * 1)(5)
    fac = (C.c_int32 * 4)(0, 1, 2, 3)
    assert L.vi_sumcheck_round(p, 16, 4, 16, 1, coefs, nfac, fac, 0, 0, p, p, None) != 0 and "factors" in _err(lib)
    nfac[0] = 2
    assert L.vi_sumcheck_round(p, 16, 4, 12, 1, coefs, nfac, fac, 0, 0, p, p, None) != 0 and "power of two" in _err(lib)
    assert L.vi_sumcheck_round(p, 16, 9, 16, 1, coefs, nfac, fac, 0, 0, p, p, None) != 0
    coins = (C.c_uint64 * 65)(*([3] * 65))
    assert L.vi_sumcheck_complete(p, 65, 3, coins, None) != 0 and "64 rounds" in _err(lib)
    assert L.vi_sumcheck_complete(p, 4, 8, coins, None) != 0 and "degree" in _err(lib)
    assert L.vi_sumcheck_complete(p, 1, 3, coins, None) == 0                   # nothing to fill
    coins[1] = (1 << 64) - 1
    assert L.vi_sumcheck_complete(p, 4, 3, coins, None) != 0 and "canonical" in _err(lib)


def test_shim_registers_reference_module_names(lib):
    from verinf_b200 import shim
    saved = {k: sys.modules.get(k) for k in ("cuda_primitives", "prover.cuda_primitives", "kquant_cuda",
                                             "prover.kquant_cuda")}
    try:
        shim.install()
        import cuda_primitives as cp
        import kquant_cuda as kq
        from verinf_b200 import cuda_primitives as mine
        assert cp is mine and sys.modules["prover.cuda_primitives"] is mine
        assert kq.QK_K == 256 and kq.BLOCK_BYTES == {"Q4_K": 144, "Q5_K": 176, "Q6_K": 210}
        # every name the reference's callers import must exist (prover/core.py:40-51 and friends)
        names = """P GLOBAL_G gl_mul gl_add gl_sub gl_neg gl_pow gl_inv gl_inv_batched gl_axpy ntt_forward
            ntt_inverse ntt_forward_batched ntt_inverse_batched rs_encode_rows poly_mul poly_add
            poly_mul_batched poly_eval gl_matmul gl_matvec gl_spmv gl_spmv_challenged challenge_vec
            challenge_at interp_band interp_band_causal_id interp_band_causal_c2 interp_band_embed
            interp_band_rope_x hash_columns_streamed merkle_build_blake3 MerkleColumnAccumulator row_prg
            row_prg_indexed lookup_multiplicities lookup_multiplicities_into""".split()
        for n in names:
            assert hasattr(cp, n), n
        assert hasattr(kq, "kquant_to_field")
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def test_python_wrappers_reject_bad_tensors_before_any_launch(lib):
    import torch
    from verinf_b200 import cuda_primitives as cp
    cpu_t = torch.zeros(8, dtype=torch.uint64)
    with pytest.raises(RuntimeError, match="CUDA"):
        cp.gl_mul(cpu_t, cpu_t)
    with pytest.raises(RuntimeError, match="CUDA"):
        cp.ntt_forward(cpu_t)
    with pytest.raises(RuntimeError):
        cp.hash_columns_streamed(cpu_t.reshape(2, 4))
    with pytest.raises(AssertionError):
        cp.MerkleColumnAccumulator(16, 128)


def test_round_sample_derivation_host_logic():
    """g(1) of a sumcheck round is derived on the host from the previous round's samples:
    check the Lagrange evaluation and the identity g_k(0) + g_k(1) = g_{k-1}(r) against the oracle"""
    import numpy as np
    import oracle
    from verinf_b200.layergkr_gpu import _interp_at, P
    rng = np.random.default_rng(0)
    coeffs = [int(v) for v in rng.integers(0, P, size=4, dtype=np.uint64)]
    poly = lambda x: sum(c * pow(x, i, P) for i, c in enumerate(coeffs)) % P
    ys = [poly(x) for x in range(4)]
    for r in (0, 3, 4, 12345678901234567, P - 1):
        assert _interp_at(ys, r) == poly(r)
    assert _interp_at([7], 99) == 7
    tabs = rng.integers(0, P, size=(3, 64), dtype=np.uint64)
    coins = [int(c) for c in rng.integers(0, P, size=6, dtype=np.uint64)]
    claim, samples, _ = oracle.sumcheck(tabs, [(1, [0, 1, 2])], coins)
    assert (int(samples[0][0]) + int(samples[0][1])) % P == claim
    for k in range(1, 6):
        prev = [int(v) for v in samples[k - 1][:4]]
        assert (int(samples[k][0]) + int(samples[k][1])) % P == _interp_at(prev, coins[k - 1])
