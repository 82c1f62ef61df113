"""Row-batch commitment: Reed-Solomon encode -> BLAKE3 column leaves -> Merkle root.

This is the hot path of the reference's commit phase (prover/core.py:1206-1320
`_stream_phase`: encode_messages -> MerkleColumnAccumulator.update -> merkle_build_blake3,
and layergkr/rs.py:195-213 `Commit.from_messages`) with buffers allocated once and reused,
so a steady-state commit issues only this library's kernels.
"""
import torch

from . import cuda_primitives as cp
from ._lib import LIB, check, ptr, stream_ptr


def _index_tensor(cols, limit, device, what):
    """host list / tensor of indices -> validated int64 device tensor"""
    t = torch.as_tensor(cols, dtype=torch.int64)
    if t.numel() and (int(t.min()) < 0 or int(t.max()) >= limit):
        raise RuntimeError(f"{what}: index outside [0, {limit})")
    return t.to(device).contiguous()


def open_columns(codes, cols, out=None, row0=0):
    """The queried columns of a (m, N) codeword matrix as a (T, total_rows) tensor, each opened
    column contiguous: out[t, row0 + r] = codes[r, cols[t]].  Replaces `codes.index_select(1, Q)`
    plus the per-column clone / cat of prover/core.py:1304-1320; with `out` and `row0` a matrix
    that arrives in row chunks fills one buffer."""
    assert codes.is_cuda and codes.dtype == torch.uint64 and codes.dim() == 2 and codes.is_contiguous()
    m, n = codes.shape
    idx = cols if (torch.is_tensor(cols) and cols.is_cuda) else _index_tensor(cols, n, codes.device, "open_columns")
    T = idx.numel()
    if out is None:
        out = torch.empty((T, row0 + m), dtype=torch.uint64, device=codes.device)
    assert out.dtype == torch.uint64 and out.is_contiguous() and out.size(0) == T
    with torch.cuda.device(codes.device):
        check(LIB.vi_open_columns(ptr(codes), m, n, ptr(idx), T, ptr(out), out.size(1), row0, stream_ptr()))
    return out


def merkle_paths(leaves, upper, idx):
    """Authentication paths of the leaves `idx` from a tree that stays on the device.
    leaves (N, 32) uint8 and upper (vi_merkle_upper_nodes(N), 32) uint8 as produced by the Merkle
    build.  Returns (siblings (T, depth, 32) uint8, sides (T, depth) uint8) on the device, with
    the convention of merkle_path (prover/core.py:305-317): level by level from the leaves, the
    sibling (the node itself where an odd level has none) and side = 1 when the path node is the
    left child."""
    assert leaves.is_cuda and leaves.dtype == torch.uint8 and leaves.is_contiguous() and leaves.size(1) == 32
    n = leaves.size(0)
    idx_t = idx if (torch.is_tensor(idx) and idx.is_cuda) else _index_tensor(idx, n, leaves.device, "merkle_paths")
    T, depth = idx_t.numel(), LIB.vi_merkle_depth(n)
    sib = torch.empty((T, depth, 32), dtype=torch.uint8, device=leaves.device)
    sides = torch.empty((T, depth), dtype=torch.uint8, device=leaves.device)
    with torch.cuda.device(leaves.device):
        check(LIB.vi_merkle_paths(ptr(leaves), n, ptr(upper), ptr(idx_t), T, ptr(sib), ptr(sides), stream_ptr()))
    return sib, sides


def paths_as_reference(siblings, sides):
    """device path tensors -> the reference's host form: one list of (sibling bytes, side) per
    query (prover/core.py:305-317); a single D2H copy of T*depth*33 bytes."""
    sib = siblings.cpu().numpy()
    sd = sides.cpu().numpy()
    return [[(sib[t, l].tobytes(), int(sd[t, l])) for l in range(sib.shape[1])] for t in range(sib.shape[0])]


class RowCommitter:
    """Commits batches of `rows` message rows (ELL values each) at geometry (K, N).

    commit(msg)       msg is a (rows, ELL) uint64 CUDA tensor; returns the 32-byte root
                      tensor (device).  Codewords stay in `self.codes`, leaves and the upper
                      tree levels in `self.leaves` / `self.upper`.
    commit_host(msg)  msg is a pinned host tensor; rows are copied in slices on a second
                      stream so the copy of slice i+1 overlaps the encode of slice i; returns
                      the root as 32 bytes on the host.
    """

    def __init__(self, rows, ell, k_deg, n_lig, *, master_seed=None, device="cuda", h2d_slices=32):
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
        self._stream_state = None
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
            # slices of whole 128-row BLAKE3 chunks are hashed as soon as they are encoded (streaming
            # column hash), so that after the last copy only one slice of work remains
            streamed = self.rows > 128 and step >= 128
            if streamed:
                step = (step // 128) * 128
                if self._stream_state is None:
                    nb = LIB.vi_hash_stream_state_bytes(self.n, self.rows)
                    self._stream_state = torch.empty(max(nb, 256), dtype=torch.uint8, device=self.device)
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
                if streamed:
                    check(LIB.vi_hash_stream_update(ptr(self._stream_state), self.n, self.rows, r0,
                                                    self.codes[r0:r0 + cnt].data_ptr(), cnt, ptr(self.leaves),
                                                    stream_ptr()))
            if streamed:
                check(LIB.vi_merkle_build(ptr(self.leaves), self.n, ptr(self.upper), stream_ptr()))
            else:
                self._hash_and_tree()
            self._root_host.copy_(self.root, non_blocking=True)
            main.synchronize()
        return bytes(self._root_host.tolist())

    def copy_only(self, msg_host):
        """The host-to-device part of commit_host alone: the same pinned rows, staging buffer, slices
        and copy stream, no kernel.  What it takes is the floor the host memory and PCIe path set for
        commit_host on this machine (used by the benchmark beside the end-to-end figure)."""
        assert not msg_host.is_cuda and msg_host.is_pinned() and tuple(msg_host.shape) == (self.rows, self.ell)
        with torch.cuda.device(self.device):
            if self._stage is None:
                self._stage = torch.empty((self.rows, self.ell), dtype=torch.uint64, device=self.device)
                self._copy_stream = torch.cuda.Stream(device=self.device)
            main = torch.cuda.current_stream()
            step = (self.rows + self._slices - 1) // self._slices
            if self.rows > 128 and step >= 128:
                step = (step // 128) * 128
            self._copy_stream.wait_stream(main)
            with torch.cuda.stream(self._copy_stream):
                for r0 in range(0, self.rows, step):
                    cnt = min(step, self.rows - r0)
                    self._stage[r0:r0 + cnt].copy_(msg_host[r0:r0 + cnt], non_blocking=True)
            main.wait_stream(self._copy_stream)
            main.synchronize()

    def open(self, cols):
        """Opening of the last commit at the queried columns: (columns (T, rows) uint64,
        siblings (T, depth, 32), sides (T, depth)), all on the device."""
        idx = _index_tensor(cols, self.n, self.device, "open")
        sib, sides = merkle_paths(self.leaves, self.upper, idx)
        return open_columns(self.codes, idx), sib, sides

    @property
    def h2d_bytes(self):
        return self.rows * self.ell * 8

    @property
    def d2h_bytes(self):
        return 32


class StreamCommitter:
    """One commitment over `total_rows` message rows that arrive in chunks, without ever holding
    the codeword matrix: each `update(chunk)` pads + encodes the chunk, feeds the column-hash
    accumulator and, when `open_cols` is given, appends the chunk's entries of those columns to a
    (T, total_rows) buffer.  `finalize()` builds the tree and returns the root.

    This is the device half of the reference's `_stream_phase` loop (prover/core.py:1206-1320:
    encode_messages -> merkle_acc.update -> codes.index_select(1, Q_set)) as one object whose
    buffers are allocated once.  Any chunk sizes are accepted; `total_rows` must exceed 128
    (as MerkleColumnAccumulator requires, prover/cuda_primitives.py:1297-1385)."""

    def __init__(self, total_rows, ell, k_deg, n_lig, *, master_seed=None, row_offset=0, open_cols=None,
                 max_chunk_rows=1024, device="cuda"):
        self.total, self.ell, self.k, self.n = int(total_rows), int(ell), int(k_deg), int(n_lig)
        self.device = torch.device(device)
        self.seed, self.row_offset = master_seed, int(row_offset)
        self.max_chunk = int(max_chunk_rows)
        with torch.cuda.device(self.device):
            self.acc = cp.MerkleColumnAccumulator(self.n, self.total)
        self.codes = torch.empty((self.max_chunk, self.n), dtype=torch.uint64, device=self.device)
        self._enc_bytes = LIB.vi_encode_scratch_bytes(self.max_chunk, self.k, self.n)
        self._enc_scratch = torch.empty(max(self._enc_bytes, 256), dtype=torch.uint8, device=self.device)
        self.cols_idx = None if open_cols is None else _index_tensor(open_cols, self.n, self.device, "open_cols")
        self.opened = None if open_cols is None else torch.empty((self.cols_idx.numel(), self.total),
                                                                  dtype=torch.uint64, device=self.device)
        self.rows_done = 0
        self.leaves = self.upper = self.root = None

    def update(self, msg):
        assert msg.is_cuda and msg.dtype == torch.uint64 and msg.is_contiguous() and msg.size(1) == self.ell
        assert self.rows_done + msg.size(0) <= self.total, "more rows than announced"
        for r0 in range(0, msg.size(0), self.max_chunk):
            part = msg[r0:r0 + self.max_chunk]
            cnt = part.size(0)
            codes = self.codes[:cnt]
            with torch.cuda.device(self.device):
                check(LIB.vi_encode_rows(ptr(part), cnt, self.ell, self.k, self.n, 1 if self.seed is not None else 0,
                                         ptr(self.seed), self.row_offset + self.rows_done, None, ptr(codes),
                                         ptr(self._enc_scratch), self._enc_bytes, stream_ptr()))
            self.acc.update(codes)
            if self.opened is not None:
                open_columns(codes, self.cols_idx, out=self.opened, row0=self.rows_done)
            self.rows_done += cnt

    def finalize(self):
        assert self.rows_done == self.total, f"expected {self.total} rows, saw {self.rows_done}"
        self.leaves = self.acc.finalize()
        self.upper = torch.empty((max(LIB.vi_merkle_upper_nodes(self.n), 1), 32), dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            check(LIB.vi_merkle_build(ptr(self.leaves), self.n, ptr(self.upper), stream_ptr()))
        self.root = self.upper[LIB.vi_merkle_upper_nodes(self.n) - 1] if self.n > 1 else self.leaves[0]
        return self.root

    def paths(self, cols=None):
        """Merkle paths of the opened columns (or of `cols`) after finalize()."""
        assert self.root is not None, "finalize() first"
        idx = self.cols_idx if cols is None else _index_tensor(cols, self.n, self.device, "paths")
        return merkle_paths(self.leaves, self.upper, idx)
