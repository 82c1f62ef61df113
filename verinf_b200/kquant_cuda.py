"""Drop-in replacement for the reference's prover/kquant_cuda.py (same names:
`kquant_to_field`, `QK_K`, `BLOCK_BYTES`), backed by libverinf_b200.so.

Raw GGUF K-quant super-block bytes (Q4_K / Q5_K / Q6_K) -> committed field integers,
bit-exact with gguf-py's dequantize followed by round-half-even(double(v) * S) and the
signed-to-field map (prover/kquant_cuda.py:42-111, prover/loader.py:52-70).

`kquant_encode_rows` is the fused form with no reference counterpart: the lift happens
inside the first pass of the Reed-Solomon encode, so lifted weights never reach HBM.
"""
import torch

from ._lib import LIB, check, ptr, scratch, stream_ptr

QK_K = 256
BLOCK_BYTES = {"Q4_K": 144, "Q5_K": 176, "Q6_K": 210}
_QTYPE = {"Q4_K": 4, "Q5_K": 5, "Q6_K": 6}


def kquant_to_field(raw_u8_cuda: torch.Tensor, qtype: str, S: int) -> torch.Tensor:
    """raw K-quant bytes (any shape, contiguous, CUDA uint8) -> flat uint64 field tensor of
    n_blocks*256 integers in stored order."""
    assert qtype in _QTYPE, f"kquant_to_field: unsupported type {qtype}"
    raw = raw_u8_cuda.reshape(-1)
    if not (raw.is_cuda and raw.dtype == torch.uint8 and raw.is_contiguous()):
        raise RuntimeError("raw must be a contiguous CUDA uint8 tensor")
    nb = raw.numel() // BLOCK_BYTES[qtype]
    if nb * BLOCK_BYTES[qtype] != raw.numel():
        raise RuntimeError(f"raw size {raw.numel()} is not a multiple of the {qtype} block size")
    out = torch.empty((nb * QK_K,), dtype=torch.uint64, device=raw.device)
    with torch.cuda.device(raw.device):
        check(LIB.vi_kquant_to_field(ptr(raw), nb, _QTYPE[qtype], float(S), ptr(out), stream_ptr()))
    return out


def kquant_encode_rows(raw_u8_cuda, qtype, S, d_out, d_in, *, ell, k_deg, n_lig, transpose=True,
                       first_row=0, n_rows=None, master_seed=None, row_offset=0,
                       need_polys=False, need_codewords=True):
    """Lift + pack + encode without materialising the lifted matrix.

    The (d_out, d_in) quantised matrix is viewed as the flat field vector the loader would
    produce (transposed to (d_in, d_out) when `transpose`, prover/loader.py:433-436), cut into
    message rows of `ell` slots (prover/core.py:389-458; the last row is zero-filled), and
    rows first_row .. first_row+n_rows-1 are encoded as by encode_messages.
    Returns (row_polys or None, codewords or None)."""
    assert qtype in _QTYPE
    raw = raw_u8_cuda.reshape(-1)
    if not (raw.is_cuda and raw.dtype == torch.uint8 and raw.is_contiguous()):
        raise RuntimeError("raw must be a contiguous CUDA uint8 tensor")
    if raw.numel() * QK_K != d_out * d_in * BLOCK_BYTES[qtype]:
        raise RuntimeError("raw size does not match d_out*d_in")
    total_rows = (d_out * d_in + ell - 1) // ell
    if n_rows is None:
        n_rows = total_rows - first_row
    dev = raw.device
    polys = torch.empty((n_rows, k_deg), dtype=torch.uint64, device=dev) if need_polys else None
    codes = torch.empty((n_rows, n_lig), dtype=torch.uint64, device=dev) if need_codewords else None
    seed = master_seed.contiguous() if master_seed is not None else None
    with torch.cuda.device(dev):
        # + the staging area of the loader: 1.25 bytes per weight (transposed) or 64 bytes per super-block
        nb = LIB.vi_encode_scratch_bytes(n_rows, k_deg, n_lig) + (d_out * d_in * 5) // 4 + 256
        s = scratch(nb, dev) if nb else None
        check(LIB.vi_kquant_encode_rows(ptr(raw), _QTYPE[qtype], float(S), d_out, d_in, int(bool(transpose)),
                                        first_row, n_rows, ell, k_deg, n_lig, 1 if seed is not None else 0,
                                        ptr(seed), int(row_offset), ptr(polys), ptr(codes), ptr(s), nb,
                                        stream_ptr()))
    return polys, codes
