"""ctypes binding of libverinf_b200.so (the C ABI declared in include/verinf_b200.h).

The library is the only compute path: if it is missing or fails to load, importing
this module raises — there is no CPU or PyTorch fallback.
"""
import ctypes as C
import os
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
SO_PATH = Path(os.environ.get("VERINF_LIB") or _HERE / "libverinf_b200.so")   # VERINF_LIB: build under test

_i64, _u64, _int, _p, _dbl = C.c_int64, C.c_uint64, C.c_int, C.c_void_p, C.c_double

# name -> (restype, argtypes); kept in one table so the symbol-export test can walk it
SIGNATURES = {
    "vi_last_error": (C.c_char_p, []),
    "vi_gl_binary": (_int, [_int, _p, _p, _p, _i64, _p]),
    "vi_gl_binary_bcast": (_int, [_int, _p, _p, _i64, _p, _i64, _p]),
    "vi_gl_neg": (_int, [_p, _p, _i64, _p]),
    "vi_gl_pow": (_int, [_p, _u64, _p, _i64, _p]),
    "vi_gl_axpy": (_int, [_p, _u64, _p, _i64, _p]),
    "vi_ntt_scratch_bytes": (_i64, [_i64, _i64]),
    "vi_ntt_batched": (_int, [_p, _i64, _i64, _int, _p, _i64, _p]),
    "vi_encode_scratch_bytes": (_i64, [_i64, _i64, _i64]),
    "vi_encode_rows": (_int, [_p, _i64, _i64, _i64, _i64, _int, _p, _i64, _p, _p, _p, _i64, _p]),
    "vi_row_prg": (_int, [_p, _i64, _p, _i64, _i64, _p, _p]),
    "vi_challenge": (_int, [_p, _p, _int, _p, _i64, _p, _p]),
    "vi_hash_columns_scratch_bytes": (_i64, [_i64, _i64]),
    "vi_hash_columns": (_int, [_p, _i64, _i64, _p, _p, _i64, _p]),
    "vi_hash_columns_noalloc_max_state_bytes": (_i64, []),
    "vi_hash_columns_noalloc": (_int, [_p, _i64, _i64, _p, _p]),
    "vi_hash_stream_state_bytes": (_i64, [_i64, _i64]),
    "vi_hash_stream_update": (_int, [_p, _i64, _i64, _i64, _p, _i64, _p, _p]),
    "vi_hash_subtree_state_bytes": (_i64, [_i64, _int]),
    "vi_hash_subtree": (_int, [_p, _i64, _i64, _i64, _int, _p, _p, _p]),
    "vi_hash_merge_subtrees": (_int, [_p, _p, _int, _i64, _p, _p]),
    "vi_merkle_upper_nodes": (_i64, [_i64]),
    "vi_merkle_build": (_int, [_p, _i64, _p, _p]),
    "vi_merkle_level": (_int, [_p, _i64, _p, _p]),
    "vi_release_tables": (_int, []),
    "vi_ntt_forward_padded": (_int, [_p, _i64, _i64, _p, _i64, _p, _i64, _p]),
    "vi_product_colsum_scratch_bytes": (_i64, [_i64, _i64]),
    "vi_product_colsum": (_int, [_p, _p, _i64, _p, _p, _p, _i64, _p, _int, _p, _i64, _p]),
    "vi_merkle_depth": (_int, [_i64]),
    "vi_merkle_paths": (_int, [_p, _i64, _p, _p, _i64, _p, _p, _p]),
    "vi_open_columns": (_int, [_p, _i64, _i64, _p, _i64, _p, _i64, _i64, _p]),
    "vi_kquant_to_field": (_int, [_p, _i64, _int, _dbl, _p, _p]),
    "vi_kquant_encode_rows": (_int, [_p, _int, _dbl, _i64, _i64, _int, _i64, _i64, _i64, _i64, _i64,
                                     _int, _p, _i64, _p, _p, _p, _i64, _p]),
    "vi_sumcheck_scratch_bytes": (_i64, []),
    "vi_sumcheck_claim": (_int, [_p, _i64, _int, _i64, _int, _p, _p, _p, _p, _p, _p]),
    "vi_sumcheck_run": (_int, [_p, _i64, _int, _i64, _int, _p, _p, _p, _p, _int, _p, _p, _p]),
    "vi_sumcheck_round": (_int, [_p, _i64, _int, _i64, _int, _p, _p, _p, _int, _u64, _p, _p, _p]),
    "vi_sumcheck_complete": (_int, [_p, _int, _int, _p, _p]),
    "vi_poly_eval": (_int, [_p, _i64, _i64, _p, _i64, _p, _p]),
    "vi_gl_matmul": (_int, [_p, _p, _p, _i64, _i64, _i64, _p]),
    "vi_gl_matmul_tc_scratch_bytes": (_i64, [_i64, _i64, _i64]),
    "vi_gl_matmul_tc": (_int, [_p, _p, _p, _i64, _i64, _i64, _p, _i64, _p]),
    "vi_gl_matmul_umma_scratch_bytes": (_i64, [_i64, _i64, _i64]),
    "vi_gl_matmul_umma": (_int, [_p, _p, _p, _i64, _i64, _i64, _p, _i64, _p, _p]),
    "vi_gl_matvec": (_int, [_p, _p, _p, _i64, _i64, _p]),
    "vi_gl_spmv": (_int, [_p, _p, _p, _p, _p, _p, _int, _p, _i64, _p]),
    "vi_lookup_multiplicities": (_int, [_p, _i64, _p, _i64, _p, _p]),
    "vi_interp_band": (_int, [_int, _p, _i64, _i64, _i64, _u64, _u64, _u64, _u64,
                              _p, _p, _p, _p, _i64, _p, _p, _int, _p]),
    "vi_profile_enable": (None, [_int]),
    "vi_profile_num_tags": (_int, []),
    "vi_profile_tag_name": (C.c_char_p, [_int]),
    "vi_profile_read": (_int, [_int, C.POINTER(_dbl), C.POINTER(_i64)]),
}


def load() -> C.CDLL:
    if not SO_PATH.exists():
        raise ImportError(
            f"{SO_PATH} is missing: build it with `python -m verinf_b200.build` "
            "(nvcc, sm_100a).  verinf_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(str(SO_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)       # AttributeError here = a symbol the header declares is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


LIB = load()


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(LIB.vi_last_error().decode(errors="replace"))


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


_scratch = {}


def scratch(nbytes: int, device, tag: str = "main") -> torch.Tensor:
    """Per-device scratch owned by torch's caching allocator (so memory accounting sees
    it); grows on demand and is reused across calls."""
    key = (torch.device(device).index, tag)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def profile_enable(on: bool) -> None:
    LIB.vi_profile_enable(int(on))


def profile_read() -> dict:
    """{kernel tag: (total device ms, launches)} for every tag with at least one launch."""
    out = {}
    for t in range(LIB.vi_profile_num_tags()):
        ms, n = _dbl(0), _i64(0)
        check(LIB.vi_profile_read(t, C.byref(ms), C.byref(n)))
        if n.value:
            out[LIB.vi_profile_tag_name(t).decode()] = (ms.value, n.value)
    return out
