"""Synthetic, seeded end-to-end workloads on top of the kernels (shapes of a Llama-2-7B decoder
layer; no checkpoint is needed).  Used by `bench.py --extra` to report the secondary figures:
fused K-quant lift + encode of one MLP weight, and commit + sumcheck of a whole layer.

Layout conventions follow the reference: dense row packing of each flattened tensor into message
rows of ELL slots (prover/core.py:389-458), production geometry ELL=8192, K=16384, N=65536 with the
row_prg pad (prover/admission.py:43), int8 values lifted with the signed-to-field map
(prover/loader.py:52-58), one deg-2 sumcheck per matmul over the projected vectors
(layergkr/full_layer.py:203-230).
"""
import time

import numpy as np
import torch

from . import cuda_primitives as cp
from . import kquant_cuda as kq
from . import layergkr_gpu as lg
from .commit import RowCommitter

P = cp.P
ELL, K_DEG, N_LIG = 8192, 16384, 65536


def _signed_to_field(t_int64):
    """int64 tensor -> uint64 field tensor, negatives as p - |v| (prover/loader.py:52-58)."""
    neg = t_int64 < 0
    out = t_int64.clone()
    out[neg] = out[neg] + (P - (1 << 64))          # two's complement of p - |v| in int64 lanes
    return out.view(torch.uint64)


def _rand_int8_field(shape, gen, dev):
    return _signed_to_field(torch.randint(-128, 128, shape, dtype=torch.int64, device=dev, generator=gen))


def _pack_rows(flat):
    """flat field vector -> (rows, ELL) message matrix, zero-filled tail (core.py:389-458)."""
    n = flat.numel()
    rows = -(-n // ELL)
    if rows * ELL == n:
        return flat.view(torch.int64).reshape(rows, ELL).view(torch.uint64)
    out = torch.zeros(rows * ELL, dtype=torch.int64, device=flat.device)
    out[:n] = flat.view(torch.int64).reshape(-1)
    return out.reshape(rows, ELL).view(torch.uint64)


def _timed(fn):
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    r = fn()
    torch.cuda.synchronize()
    return r, time.perf_counter() - t0


def kquant_fused_encode(dev, qtype="Q4_K", seed=3, check_rows=None):
    """Fused lift + encode workload: 11008x4096 weight as K-quant super-blocks -> lifted and RS-encoded
    (transposed view, 5504 rows).  Compares the fused op with lift + transpose + pack + encode.
    With `check_rows` (row indices, negative = from the end) the result also carries, under "_check",
    the raw super-blocks and those codeword rows on the host for an independent checker."""
    d_out, d_in = 11008, 4096
    nb = d_out * d_in // 256
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, size=(nb, kq.BLOCK_BYTES[qtype]), dtype=np.uint8)
    scale = np.clip(rng.normal(0, 0.02, size=(nb, 2)), -6e4, 6e4).astype(np.float16).view(np.uint8).reshape(nb, 4)
    if qtype == "Q6_K":
        raw[:, 208:210] = scale[:, :2]
    else:
        raw[:, 0:4] = scale
    raw_t = torch.from_numpy(raw).to(dev)
    seed_t = torch.arange(32, dtype=torch.uint8, device=dev)
    S = 1 << 12

    def unfused():
        w = kq.kquant_to_field(raw_t, qtype, S)
        wt = w.view(torch.int64).view(d_out, d_in).T.contiguous().view(torch.uint64).reshape(-1)
        return cp.encode_rows(_pack_rows(wt), K_DEG, N_LIG, master_seed=seed_t, need_polys=False)[1]

    def fused():
        return kq.kquant_encode_rows(raw_t, qtype, S, d_out, d_in, ell=ELL, k_deg=K_DEG, n_lig=N_LIG,
                                     transpose=True, master_seed=seed_t)[1]

    a, b = unfused(), fused()
    same = bool(torch.equal(a.view(torch.int64), b.view(torch.int64)))
    rows = b.size(0)
    chk = None
    if check_rows is not None:
        idx = sorted({int(i) % rows for i in check_rows})
        sel = b.view(torch.int64)[torch.tensor(idx, device=dev)].cpu().numpy().view(np.uint64)
        chk = {"raw": raw, "rows": idx, "codes": sel, "seed": bytes(range(32)), "S": S, "d_out": d_out, "d_in": d_in,
               "ell": ELL, "k": K_DEG, "n": N_LIG}
    del a, b
    t_unf = _event_ms(unfused, reps=3, warm=1)
    t_fus = _event_ms(fused, reps=3, warm=1)
    out = {"qtype": qtype, "rows": rows, "bit_identical_to_unfused": same, "fused_ms": t_fus,
           "unfused_ms": t_unf, "encoded_elems_per_s": rows * N_LIG / t_fus * 1e3,
           "codeword_gbs": rows * N_LIG * 8 / t_fus / 1e6}
    if chk is not None:
        out["_check"] = chk
    return out


def _event_ms(fn, reps=5, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def field_matmul(dev, m=1000, k=4096, n=11008, seed=5):
    """Witness matmul Y = X W mod p of one MLP projection (gl_matmul, prover/cuda_primitives.py:1086-1106)."""
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    X = _rand_int8_field((m, k), g, dev)
    W = _rand_int8_field((k, n), g, dev)
    ms = _event_ms(lambda: cp.gl_matmul(X, W))
    out = {"m": m, "k": k, "n": n, "ms": ms, "multiply_adds_per_s": m * k * n / ms * 1e3}
    if m > 4 and n > 1:
        out["mma_sync_ms"] = _event_ms(lambda: cp.gl_matmul(X, W, path="mma"))
        out["tcgen05_ms"] = _event_ms(lambda: cp.gl_matmul(X, W, path="umma"))
        cp.check_async_errors()
    return out


def fold_products(dev, rows=1024, k_deg=K_DEG, seed=9):
    """Evaluation-domain fold of `rows` pairs of degree-<K polynomials (the q_lin / p_0 transform,
    prover/core.py:1892-1911): the fused path against the reference's sequence on the same kernels."""
    from . import fold
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    A = torch.randint(0, 1 << 62, (rows, k_deg), dtype=torch.int64, device=dev, generator=g).view(torch.uint64)
    B = torch.randint(0, 1 << 62, (rows, k_deg), dtype=torch.int64, device=dev, generator=g).view(torch.uint64)
    n_eval = fold.eval_size(k_deg)
    ones = torch.ones(rows, dtype=torch.int64, device=dev).view(torch.uint64)

    def composed():
        a_pad = A.new_zeros((rows, n_eval)); a_pad[:, :k_deg] = A
        b_pad = B.new_zeros((rows, n_eval)); b_pad[:, :k_deg] = B
        cp.ntt_forward_batched(a_pad); cp.ntt_forward_batched(b_pad)
        prod = cp.gl_mul(a_pad, b_pad)
        return cp.gl_matvec(prod.view(torch.int64).T.contiguous().view(torch.uint64), ones)

    same = bool(torch.equal(composed().view(torch.int64), fold.fold_products_eval(A, B).view(torch.int64)))
    t_ref = _event_ms(composed)
    t_fused = _event_ms(lambda: fold.fold_products_eval(A, B))
    EA, EB = fold.ntt_forward_padded(A, n_eval), fold.ntt_forward_padded(B, n_eval)
    t_sum = _event_ms(lambda: fold.product_colsum(EA, EB))
    return {"rows": rows, "K": k_deg, "n_eval": n_eval, "bit_identical_to_composed": same, "fused_ms": t_fused,
            "composed_ms": t_ref, "colsum_ms": t_sum, "colsum_gbs": 2 * rows * n_eval * 8 / t_sum / 1e6}


def layer7b_commit_sumcheck(dev, seq=1000, seed=11, with_check=False):
    """Full-layer workload (dense row packing): int8 weights/activations of one Llama-2-7B-shaped layer,
    every weight and activation tensor committed (encode + column hash + Merkle), one deg-2
    sumcheck per matmul on the projected vectors, challenges drawn from a seeded transcript before
    each sumcheck starts (layergkr/full_layer.py:221-224).  Returns stage seconds; with `with_check`
    also, under "_check", what an independent checker needs to recompute the W_Q commitment and the
    W_Q sumcheck transcript on the host."""
    from .transcript import Transcript
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    d, dff = 4096, 11008
    shapes = {"W_Q": (d, d), "W_K": (d, d), "W_V": (d, d), "W_O": (d, d), "W_gate": (d, dff), "W_up": (d, dff),
              "W_down": (dff, d)}
    W = {k: _rand_int8_field(s, g, dev) for k, s in shapes.items()}
    X = {k: _rand_int8_field((seq, s[0]), g, dev) for k, s in shapes.items()}      # input of each matmul
    (Y, t_mm) = _timed(lambda: {k: cp.gl_matmul(X[k], W[k]) for k in shapes})
    seed_t = torch.arange(32, dtype=torch.uint8, device=dev)
    committers = {}

    def commit(t, row_off):
        msg = _pack_rows(t.reshape(-1))
        c = committers.get(msg.size(0))
        if c is None:
            c = committers[msg.size(0)] = RowCommitter(msg.size(0), ELL, K_DEG, N_LIG, master_seed=seed_t, device=dev)
        return bytes(c.commit(msg.contiguous(), row_offset=row_off).cpu().tolist()), msg.size(0)

    def commit_all():
        roots, rows, off = {}, 0, 0
        for name, t in list(W.items()) + [("X_" + k, v) for k, v in X.items()] + [("Y_" + k, v) for k, v in Y.items()]:
            roots[name], r = commit(t, off)
            rows += r
            off += r
        return roots, rows

    commit_all()                                                  # warm-up (tables, allocator)
    (roots, n_rows), t_commit = _timed(commit_all)

    def sumchecks(collect=None):
        ok = True
        tr = Transcript(b"bench/layer7b")
        tr.absorb("seed", int(seed).to_bytes(8, "little"))
        for name in shapes:
            n_in, n_out = shapes[name]
            rho = _rand_int8_field((seq,), g, dev)
            tau = _rand_int8_field((n_out,), g, dev)
            a = cp.gl_matmul(rho.reshape(1, -1), X[name])[0]                                          # rho^T X  (n_in), X streamed once
            b = cp.gl_matvec(W[name], tau)                                                            # W tau    (n_in)
            width = 1 << (n_in - 1).bit_length()
            fa = torch.zeros(width, dtype=torch.int64, device=dev); fa[:n_in] = a.view(torch.int64)
            fb = torch.zeros(width, dtype=torch.int64, device=dev); fb[:n_in] = b.view(torch.int64)
            # the challenges of a layergkr sumcheck are drawn before it starts
            # (layergkr/full_layer.py:222 `coins = tr.coin(f"sc_{m.name}", n)`), so all rounds are queued at once
            coins = tr.coin(f"sc_{name}", width.bit_length() - 1)
            claim, polys, _, _ = lg.prove_terms_gpu([(1, [fa.view(torch.uint64), fb.view(torch.uint64)])],
                                                    lambda i: coins[i], coins=coins)
            yt = cp.gl_matvec(Y[name], tau)                                                           # Y tau (seq)
            want = int(cp.gl_matvec(yt.reshape(1, -1), rho)[0].item())                                # rho^T Y tau
            ok = ok and claim == want and (polys[0][0][1] + polys[0][1][1]) % P == claim
            if collect is not None and name == "W_Q":
                to_np = lambda t: t.view(torch.int64).cpu().numpy().view(np.uint64)
                collect.update(rho=to_np(rho), tau=to_np(tau), coins=list(coins), claim=int(claim),
                               polys=[[int(y) for _, y in rp] for rp in polys])
        return ok

    sumchecks()
    chk = {} if with_check else None
    ok, t_sc = _timed(lambda: sumchecks(chk))
    out = {"seq": seq, "rows_committed": n_rows, "codeword_gb": n_rows * N_LIG * 8 / 1e9,
           "commit_s": t_commit, "sumcheck_s": t_sc, "commit_plus_sumcheck_s": t_commit + t_sc,
           "witness_matmul_s": t_mm, "sumcheck_claims_match_rho_Y_tau": bool(ok),
           "root_W_Q": roots["W_Q"].hex()}
    if with_check:
        to_np = lambda t: t.view(torch.int64).cpu().numpy().view(np.uint64)
        chk.update(W_Q=to_np(W["W_Q"]), X_Q=to_np(X["W_Q"]), seed=bytes(range(32)), root_W_Q=roots["W_Q"],
                   ell=ELL, k=K_DEG, n=N_LIG)
        out["_check"] = chk
    return out


def moe_expert_commits(dev, experts, d_ff=5120, d_model=8192, chunk_rows=1024, seed=17, prefix_check=False):
    """MoE variant of the full layer (layergkr/full_layer.py:245-263): every expert weight
    (d_ff x d_model int8, lifted with the signed-to-field map) gets its own commitment.  `experts` is the
    list of expert indices this process commits (16 per GPU when 128 experts are split over 8 GPUs).
    The 5120 message rows of an expert are generated and committed in chunks of `chunk_rows` through
    StreamCommitter, so neither the lifted weight nor its codeword matrix is ever held.  Expert e's
    data depends on (seed, e) only, so roots do not depend on how experts are split over processes.
    Returns seconds, rows, and the roots; with `prefix_check` also the first chunk of the first expert
    and the root of that chunk committed alone (for an independent checker)."""
    from .commit import StreamCommitter
    rows_per_expert = -(-(d_ff * d_model) // ELL)
    seed_t = torch.arange(32, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev)

    def expert_chunks(e):
        g.manual_seed(seed * 1000003 + e)
        left = d_ff * d_model
        while left > 0:
            n = min(left, chunk_rows * ELL)
            flat = _signed_to_field(torch.randint(-128, 128, (n,), dtype=torch.int64, device=dev, generator=g))
            yield _pack_rows(flat)
            left -= n

    def commit_expert(e):
        sc = StreamCommitter(rows_per_expert, ELL, K_DEG, N_LIG, master_seed=seed_t, max_chunk_rows=chunk_rows,
                             device=dev)
        for chunk in expert_chunks(e):
            sc.update(chunk.contiguous())
        return bytes(sc.finalize().cpu().tolist())

    if experts:
        commit_expert(experts[0])                      # warm-up: tables, allocator
    (roots, dt) = _timed(lambda: [commit_expert(e) for e in experts])
    out = {"experts": list(experts), "rows": rows_per_expert * len(experts), "seconds": dt, "roots": roots,
           "codeword_gb": rows_per_expert * len(experts) * N_LIG * 8 / 1e9}
    if prefix_check and experts:
        first = next(expert_chunks(experts[0])).contiguous()
        root, _, _ = cp.commit_rows(first, K_DEG, N_LIG, master_seed=seed_t)
        out["_check"] = {"msg": first.view(torch.int64).cpu().numpy().view(np.uint64), "seed": bytes(range(32)),
                         "root": bytes(root.cpu().tolist()), "k": K_DEG, "n": N_LIG, "ell": ELL}
    return out
