"""Row-batch commitment: Reed-Solomon encode -> BLAKE3 column leaves -> Merkle root.

This is the hot path of the reference's commit phase (prover/core.py:1206-1320
`_stream_phase`: encode_messages -> MerkleColumnAccumulator.update -> merkle_build_blake3,
and layergkr/rs.py:195-213 `Commit.from_messages`) with buffers allocated once and reused,
so a steady-state commit issues only this library's kernels.
"""
import torch

from . import cuda_primitives as cp
from ._lib import LIB, check, ptr, stream_ptr


class RowCommitter:
    """Commits batches of `rows` message rows (ELL values each) at geometry (K, N).

    commit(msg)       msg is a (rows, ELL) uint64 CUDA tensor; returns the 32-byte root
                      tensor (device).  Codewords stay in `self.codes`, leaves and the upper
                      tree levels in `self.leaves` / `self.upper`.
    commit_host(msg)  msg is a pinned host tensor; rows are copied in slices on a second
                      stream so the copy of slice i+1 overlaps the encode of slice i; returns
                      the root as 32 bytes on the host.
    """

    def __init__(self, rows, ell, k_deg, n_lig, *, master_seed=None, device="cuda", h2d_slices=8):
        self.rows, self.ell, self.k, self.n = int(rows), int(ell), int(k_deg), int(n_lig)
        self.device = torch.device(device)
        self.seed = master_seed
        dev = self.device
        self.codes = torch.empty((self.rows, self.n), dtype=torch.uint64, device=dev)
        self.leaves = torch.empty((self.n, 32), dtype=torch.uint8, device=dev)
        self.upper = torch.empty((max(LIB.vi_merkle_upper_nodes(self.n), 1), 32), dtype=torch.uint8, device=dev)
        self._enc_bytes = LIB.vi_encode_scratch_bytes(self.rows, self.k, self.n)
        self._enc_scratch = torch.empty(max(self._enc_bytes, 256), dtype=torch.uint8, device=dev)
        self._hash_bytes = LIB.vi_hash_columns_scratch_bytes(self.rows, self.n)
        self._hash_scratch = torch.empty(max(self._hash_bytes, 256), dtype=torch.uint8, device=dev)
        self._stage = None
        self._copy_stream = None
        self._slices = max(1, int(h2d_slices))
        self._root_host = torch.empty(32, dtype=torch.uint8).pin_memory() if dev.type == "cuda" else None

    @property
    def root(self):
        return self.upper[LIB.vi_merkle_upper_nodes(self.n) - 1] if self.n > 1 else self.leaves[0]

    def _encode(self, src_rows, r0, cnt, row_offset):
        """encode `cnt` message rows starting at device pointer `src_rows` into codeword rows r0.."""
        check(LIB.vi_encode_rows(src_rows, cnt, self.ell, self.k, self.n, 1 if self.seed is not None else 0,
                                 ptr(self.seed), row_offset + r0, None, self.codes[r0:r0 + cnt].data_ptr(),
                                 ptr(self._enc_scratch), self._enc_bytes, stream_ptr()))

    def _hash_and_tree(self):
        check(LIB.vi_hash_columns(ptr(self.codes), self.rows, self.n, ptr(self.leaves),
                                  ptr(self._hash_scratch), self._hash_bytes, stream_ptr()))
        check(LIB.vi_merkle_build(ptr(self.leaves), self.n, ptr(self.upper), stream_ptr()))

    def commit(self, msg, row_offset=0):
        assert msg.is_cuda and msg.dtype == torch.uint64 and msg.is_contiguous()
        assert tuple(msg.shape) == (self.rows, self.ell)
        with torch.cuda.device(self.device):
            self._encode(msg.data_ptr(), 0, self.rows, row_offset)
            self._hash_and_tree()
        return self.root

    def commit_host(self, msg_host, row_offset=0):
        assert not msg_host.is_cuda and msg_host.is_pinned() and msg_host.dtype == torch.uint64
        assert tuple(msg_host.shape) == (self.rows, self.ell)
        with torch.cuda.device(self.device):
            if self._stage is None:
                self._stage = torch.empty((self.rows, self.ell), dtype=torch.uint64, device=self.device)
                self._copy_stream = torch.cuda.Stream(device=self.device)
            main = torch.cuda.current_stream()
            step = (self.rows + self._slices - 1) // self._slices
            self._copy_stream.wait_stream(main)       # previous commit no longer reads the staging buffer
            events = []
            with torch.cuda.stream(self._copy_stream):
                for r0 in range(0, self.rows, step):
                    cnt = min(step, self.rows - r0)
                    self._stage[r0:r0 + cnt].copy_(msg_host[r0:r0 + cnt], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self._copy_stream)
                    events.append((r0, cnt, ev))
            for r0, cnt, ev in events:
                main.wait_event(ev)
                self._encode(self._stage[r0:r0 + cnt].data_ptr(), r0, cnt, row_offset)
            self._hash_and_tree()
            self._root_host.copy_(self.root, non_blocking=True)
            main.synchronize()
        return bytes(self._root_host.tolist())

    @property
    def h2d_bytes(self):
        return self.rows * self.ell * 8

    @property
    def d2h_bytes(self):
        return 32
