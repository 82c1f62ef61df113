"""Registers the drop-in modules under the names the reference's callers import.

The reference binds to its CUDA layer by module name — `from cuda_primitives import ...`
with prover/ pushed to sys.path[0], `from kquant_cuda import kquant_to_field`, and
`from prover import cuda_primitives as cp` in layergkr — so path order cannot win.
`install()` pre-registers this package's modules in sys.modules under all four names;
call it before importing any reference module and the untouched core.py / tape.py /
layergkr pick up the sm_100a kernels.
"""
import sys


def install() -> None:
    from . import cuda_primitives, kquant_cuda
    for name in ("cuda_primitives", "prover.cuda_primitives"):
        sys.modules[name] = cuda_primitives
    for name in ("kquant_cuda", "prover.kquant_cuda"):
        sys.modules[name] = kquant_cuda
    pkg = sys.modules.get("prover")
    if pkg is not None:
        pkg.cuda_primitives = cuda_primitives
        pkg.kquant_cuda = kquant_cuda


_LAYERGKR_FAST = ("encode_batch_ntt", "hash_and_tree", "prove_terms_gpu", "combine_t", "encode_batch_t",
                  "gl_sum", "fold_t")


def install_layergkr() -> None:
    """Optional second step, after install() and with the reference's root on sys.path: replaces the
    device routines of the reference's `layergkr.gpu` module (layergkr/gpu.py:141-410) by this
    package's fused versions (one encode call, one fold+evaluate launch per sumcheck round).  The
    module itself, its self-tests and every caller (`rs.py`, `sumcheck.py`, `layer.py`, ...) stay the
    reference's: they look the routines up in `layergkr.gpu` by name."""
    import importlib
    from . import layergkr_gpu
    import functools
    gpu = importlib.import_module("layergkr.gpu")
    for name in _LAYERGKR_FAST:
        setattr(gpu, name, getattr(layergkr_gpu, name))
    # every sumcheck call site of the reference draws its challenges before the sumcheck starts and hands
    # over `lambda i: coins[i]` (layergkr/relations.py:122-123, layergkr/sumcheck.py:146), so the rounds can
    # be queued without a host round trip each
    gpu.prove_terms_gpu = functools.partial(layergkr_gpu.prove_terms_gpu, predraw=True)
