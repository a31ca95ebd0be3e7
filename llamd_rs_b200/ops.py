"""Device-pointer ops of the C ABI, wrapped for numpy in / numpy out.

The counterpart of ``llamd_rocm::op`` (crates/llamd-rocm/src/forward.rs:733-1676):
each function checks sizes before the FFI call, uploads its inputs, queues the
op on the library stream, synchronises and downloads the result. Meant for
tests and experiments; the resident model (``model.CudaModel``) chains the same
entry points without leaving the device.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import backend
from ._lib import lib
from .backend import DevBuf, Malformed, ShapeError

QK_K = 256


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def quantize(x):
    """f32 [n] -> (qs int8[n], d f32[n/256]) on the device (op::quantize)."""
    x = _f32(x).ravel()
    if x.size == 0 or x.size % QK_K:
        raise Malformed(f"q8k input: {x.size} is not a multiple of {QK_K}")
    nb = x.size // QK_K
    dx, dq, dd = DevBuf.from_array(x), DevBuf(x.size), DevBuf(nb * 4)
    lib().llamd_fwd_quantize(dx.ptr, dq.ptr, dd.ptr, nb)
    backend.sync()
    return dq.download(np.int8, x.size), dd.download_f32(nb)


def rms_norm_mul(x, w, eps: float):
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    w = _f32(w).ravel()
    if w.size != x2.shape[1]:
        raise ShapeError(f"weight of {w.size} for rows of {x2.shape[1]}")
    dx, dw, do = DevBuf.from_array(x2), DevBuf.from_array(w), DevBuf(x2.nbytes)
    lib().llamd_fwd_rms_norm_mul(dx.ptr, dw.ptr, do.ptr, x2.shape[1], eps, x2.shape[0])
    backend.sync()
    return do.download_f32(x2.size).reshape(x.shape)


def rms_norm_quant(x, w, eps: float, residual=None):
    """-> (out f32, qs, d[, x+residual])"""
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    n, nseq = x2.shape[1], x2.shape[0]
    w = _f32(w).ravel()
    if w.size != n or n % QK_K:
        raise ShapeError(f"weight of {w.size} for rows of {n}")
    dx, dw, do = DevBuf.from_array(x2), DevBuf.from_array(w), DevBuf(x2.nbytes)
    dq, dd = DevBuf(x2.size), DevBuf(nseq * (n // QK_K) * 4)
    if residual is None:
        lib().llamd_fwd_rms_norm_quant(dx.ptr, dw.ptr, do.ptr, dq.ptr, dd.ptr, n, eps, nseq)
        backend.sync()
        return do.download_f32(x2.size).reshape(x.shape), dq.download(np.int8, x2.size), dd.download_f32(nseq * (n // QK_K))
    r = _f32(residual).reshape(x2.shape)
    dr, ds = DevBuf.from_array(r), DevBuf(x2.nbytes)
    lib().llamd_fwd_add_rms_norm_quant(dx.ptr, dr.ptr, ds.ptr, dw.ptr, do.ptr, dq.ptr, dd.ptr, n, eps, nseq)
    backend.sync()
    return (do.download_f32(x2.size).reshape(x.shape), dq.download(np.int8, x2.size), dd.download_f32(nseq * (n // QK_K)),
            ds.download_f32(x2.size).reshape(x.shape))


def head_rms_norm_mul(x, w, n_head: int, hd: int, eps: float):
    x, w = _f32(x).ravel(), _f32(w).ravel()
    if x.size != n_head * hd or w.size != hd:
        raise ShapeError("head_rms_norm_mul sizes")
    dx, dw, do = DevBuf.from_array(x), DevBuf.from_array(w), DevBuf(x.nbytes)
    lib().llamd_fwd_head_rms_norm_mul(dx.ptr, dw.ptr, do.ptr, n_head, hd, eps)
    backend.sync()
    return do.download_f32(x.size)


def rope_table(max_pos: int, hd: int, freq_base: float) -> np.ndarray:
    tab = np.zeros((max_pos, hd // 2, 2), dtype=np.float32)
    if lib().llamd_cuda_rope_table(tab.ctypes.data_as(C.c_void_p), max_pos, hd, freq_base) != 0:
        raise Malformed("rope table arguments")
    return tab


def norm_rope(x, w, n_head: int, hd: int, pos: int, freq_base: float, eps: float):
    """Per-head RMS norm (w may be None) then NeoX RoPE at `pos` (op::norm_rope)."""
    x = _f32(x).ravel()
    if x.size != n_head * hd:
        raise ShapeError("norm_rope sizes")
    tab = DevBuf.from_array(rope_table(pos + 1, hd, freq_base))
    meta = DevBuf.from_array(np.array([0, pos], np.int32))
    dx = DevBuf.from_array(x)
    dw = DevBuf.from_array(_f32(w)) if w is not None else None
    lib().llamd_fwd_norm_rope(dx.ptr, dw.ptr if dw else None, n_head, hd, meta.ptr, tab.ptr, eps, 1)
    backend.sync()
    return dx.download_f32(x.size)


def attention(q, k, v, n_kv: int, n_head: int, n_head_kv: int, hd: int, scores: bool = False):
    """scores=True hands the kernel a scores scratch buffer, which selects the
    variant that splits each head over several CTAs."""
    q, k, v = _f32(q).ravel(), _f32(k).ravel(), _f32(v).ravel()
    # same order of checks as attend (crates/llamd-runtime/src/attention.rs:63-85)
    if n_head_kv == 0 or n_head % n_head_kv:
        raise Malformed(f"attention: {n_head} query heads do not group into {n_head_kv} kv heads")
    if hd == 0:
        raise Malformed("attention: head_dim is zero")
    if q.size != n_head * hd or k.size != n_kv * n_head_kv * hd or v.size != k.size:
        raise ShapeError("attention sizes")
    if n_kv == 0:
        raise Malformed("attention: nothing to attend to")
    dq, dk, dv, do = DevBuf.from_array(q), DevBuf.from_array(k), DevBuf.from_array(v), DevBuf(q.nbytes)
    ds = DevBuf(n_head * n_kv * 4) if scores else None
    lib().llamd_fwd_attention(dq.ptr, dk.ptr, dv.ptr, do.ptr, ds.ptr if ds else None, n_head, n_head_kv, hd, n_kv)
    backend.sync()
    return do.download_f32(q.size)


def attention_prefill(q, k, v, positions, n_head: int, n_head_kv: int, hd: int, max_kv: int, tiled: bool = True):
    """One query per tile token: token i (position positions[i]) attends rows 0..positions[i] of the ONE cache
    k/v ([n_rows][n_head_kv*hd]). tiled=False runs the per-token kernels on the same inputs."""
    q, k, v = _f32(q).ravel(), _f32(k).ravel(), _f32(v).ravel()
    positions = np.ascontiguousarray(positions, dtype=np.int32).ravel()
    ntok, kv_dim = positions.size, n_head_kv * hd
    if n_head_kv == 0 or n_head % n_head_kv:
        raise Malformed(f"attention: {n_head} query heads do not group into {n_head_kv} kv heads")
    if q.size != ntok * n_head * hd or k.size != v.size or k.size % kv_dim or k.size // kv_dim > max_kv:
        raise ShapeError("attention_prefill sizes")
    if ntok == 0 or positions.min() < 0 or positions.max() >= k.size // kv_dim:
        raise Malformed("attention_prefill: a position outside the cache")
    meta = np.zeros((ntok, 2), dtype=np.int32)
    meta[:, 1] = positions
    dq, dk, dv, do = DevBuf.from_array(q), DevBuf.from_array(k), DevBuf.from_array(v), DevBuf(q.nbytes)
    dm, ds = DevBuf.from_array(meta), DevBuf(ntok * n_head * max_kv * 4)
    if tiled:
        lib().llamd_fwd_attention_prefill(dq.ptr, dk.ptr, dv.ptr, do.ptr, ds.ptr, n_head, n_head_kv, hd, dm.ptr, max_kv, ntok,
                                          int(positions.max()) + 1)
    else:
        lib().llamd_fwd_attention_tile(dq.ptr, dk.ptr, dv.ptr, do.ptr, ds.ptr, n_head, n_head_kv, hd, dm.ptr, max_kv, ntok)
    backend.sync()
    return do.download_f32(q.size).reshape(ntok, n_head * hd)


def silu_mul_quant(gate, up):
    gate, up = _f32(gate).ravel(), _f32(up).ravel()
    if gate.size != up.size or gate.size % QK_K:
        raise ShapeError("silu_mul_quant sizes")
    n = gate.size
    dg, du, do, dq, dd = DevBuf.from_array(gate), DevBuf.from_array(up), DevBuf(n * 4), DevBuf(n), DevBuf(n // QK_K * 4)
    lib().llamd_fwd_silu_mul_quant(dg.ptr, du.ptr, do.ptr, dq.ptr, dd.ptr, n)
    backend.sync()
    return do.download_f32(n), dq.download(np.int8, n), dd.download_f32(n // QK_K)


def silu_mul(gate, up):
    gate, up = _f32(gate).ravel(), _f32(up).ravel()
    if gate.size != up.size:
        raise ShapeError("silu_mul sizes")
    dg, du, do = DevBuf.from_array(gate), DevBuf.from_array(up), DevBuf(max(gate.nbytes, 4))
    lib().llamd_fwd_silu_mul(dg.ptr, du.ptr, do.ptr, gate.size)
    backend.sync()
    return do.download_f32(gate.size)


def expf(x):
    """The library's exponential, elementwise: bit for bit the host libm's expf (llamd_fwd_expf)."""
    x = _f32(x).ravel()
    dx, do = DevBuf.from_array(x), DevBuf(max(x.nbytes, 4))
    lib().llamd_fwd_expf(dx.ptr, do.ptr, x.size)
    backend.sync()
    return do.download_f32(x.size)


def router(logits, n_used: int):
    """-> (ids int32 [nseq][n_used], weights, probs) (op::router)."""
    logits = _f32(logits)
    l2 = logits.reshape(-1, logits.shape[-1])
    nseq, ne = l2.shape
    if n_used == 0 or n_used > ne:
        raise Malformed(f"moe routing: {n_used} experts requested of {ne}")
    dl, di, dw, dp = DevBuf.from_array(l2), DevBuf(nseq * n_used * 4), DevBuf(nseq * n_used * 4), DevBuf(l2.nbytes)
    lib().llamd_fwd_router(dl.ptr, ne, n_used, di.ptr, dw.ptr, dp.ptr, nseq)
    backend.sync()
    return (di.download_i32(nseq * n_used).reshape(nseq, n_used), dw.download_f32(nseq * n_used).reshape(nseq, n_used),
            dp.download_f32(l2.size).reshape(nseq, ne))


def router_matvec(w, x, n_used: int):
    """Router matrix f32 [n_expert][k] and activations [nseq][k] -> (logits, ids, weights)."""
    w, x = _f32(w), _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    ne, k = w.shape
    nseq = x2.shape[0]
    if x2.shape[1] != k:
        raise ShapeError("router_matvec sizes")
    if n_used == 0 or n_used > ne:
        raise Malformed(f"moe routing: {n_used} experts requested of {ne}")
    dw_, dx = DevBuf.from_array(w), DevBuf.from_array(x2)
    dl, di, dwt, dc = DevBuf(nseq * ne * 4), DevBuf(nseq * n_used * 4), DevBuf(nseq * n_used * 4), DevBuf.zeroed(4 * nseq)
    lib().llamd_fwd_router_matvec(dw_.ptr, dx.ptr, k, ne, n_used, dl.ptr, di.ptr, dwt.ptr, None, dc.ptr, nseq)
    backend.sync()
    assert not dc.download(np.uint32, nseq).any(), "arrival counters must return to zero"
    return (dl.download_f32(nseq * ne).reshape(nseq, ne), di.download_i32(nseq * n_used).reshape(nseq, n_used),
            dwt.download_f32(nseq * n_used).reshape(nseq, n_used))


def matvec_f32(w, x):
    w, x = _f32(w), _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    rows, k = w.shape
    if x2.shape[1] != k:
        raise ShapeError("matvec_f32 sizes")
    dw_, dx, do = DevBuf.from_array(w), DevBuf.from_array(x2), DevBuf(x2.shape[0] * rows * 4)
    lib().llamd_fwd_matvec_f32_batch(dw_.ptr, dx.ptr, do.ptr, k, rows, x2.shape[0])
    backend.sync()
    return do.download_f32(x2.shape[0] * rows).reshape(x2.shape[0], rows)


def matmul_f32_tokens(w, x):
    """The f32 matvec for every token of a tile in one launch: w [rows][k], x [ntok][k] -> [ntok][rows]."""
    w, x = _f32(w), _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    rows, k = w.shape
    if x2.shape[1] != k or k % 4:
        raise ShapeError("matmul_f32_tokens sizes")
    dw_, dx, do = DevBuf.from_array(w), DevBuf.from_array(x2), DevBuf(x2.shape[0] * rows * 4)
    lib().llamd_fwd_matmul_f32_tokens(dw_.ptr, dx.ptr, do.ptr, k, rows, x2.shape[0])
    backend.sync()
    return do.download_f32(x2.shape[0] * rows).reshape(x2.shape[0], rows)


def moe_combine_add(down, weights, residual):
    """down [nseq][n_used][n_embd], weights [nseq][n_used], residual [nseq][n_embd] or None."""
    down, weights = _f32(down), _f32(weights)
    nseq, nu, E = down.shape
    if weights.shape != (nseq, nu):
        raise ShapeError("moe_combine sizes")
    dd, dw_, do = DevBuf.from_array(down), DevBuf.from_array(weights), DevBuf(nseq * E * 4)
    dr = DevBuf.from_array(_f32(residual).reshape(nseq, E)) if residual is not None else None
    lib().llamd_fwd_moe_combine_add(dd.ptr, dw_.ptr, dr.ptr if dr else None, do.ptr, nu, E, nseq)
    backend.sync()
    return do.download_f32(nseq * E).reshape(nseq, E)


def argmax(x, nblocks: int = 512):
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    nseq, n = x2.shape
    dx, sv, si, do = DevBuf.from_array(x2), DevBuf(nblocks * nseq * 4), DevBuf(nblocks * nseq * 4), DevBuf(4 * nseq)
    lib().llamd_fwd_argmax(dx.ptr, n, sv.ptr, si.ptr, do.ptr, nblocks, nseq)
    backend.sync()
    return do.download_i32(nseq)


def moe_group(ids, n_expert: int, n_used: int):
    """ids int32 [nseq][n_used] -> dict(gstart, gcount, ptoken, pslot, work [n_work][3])."""
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    nseq = ids.size // n_used
    npair = nseq * n_used
    di = DevBuf.from_array(ids)
    gs, gc = DevBuf(n_expert * 4), DevBuf(n_expert * 4)
    pt, ps = DevBuf(max(npair, 1) * 4), DevBuf(max(npair, 1) * 4)
    wk, nw = DevBuf((npair // 8 + n_expert + 1) * 12), DevBuf.zeroed(4)
    lib().llamd_fwd_moe_group_work(di.ptr, n_expert, n_used, nseq, gs.ptr, gc.ptr, pt.ptr, ps.ptr, wk.ptr, nw.ptr)
    backend.sync()
    n_work = int(nw.download_i32(1)[0])
    return dict(gstart=gs.download_i32(n_expert), gcount=gc.download_i32(n_expert), ptoken=pt.download_i32(npair),
                pslot=ps.download_i32(npair), work=wk.download_i32(3 * n_work).reshape(n_work, 3))


def embed(table: "backend.DeviceWeights", token: int) -> np.ndarray:
    if token < 0 or token >= table.rows():
        raise Malformed(f"get_rows: id {token} is outside a table of {table.rows()} rows")
    do = DevBuf(table.blocks() * QK_K * 4)
    lib().llamd_fwd_embed(table.ptr, token, do.ptr, table.blocks())
    backend.sync()
    return do.download_f32(table.blocks() * QK_K)


def _tc_check():
    st = lib().llamd_fwd_gemm_tc_status()
    if st != 0:
        raise backend.Other(f"tcgen05 GEMM: a wait ran out (status {st})")


def matvec_tokens(weights, x, gemm=False):
    """`weights`: 1-3 DeviceWeights sharing the column count; x f32 [ntok][k].
    Quantizes on the device, then every token against every matrix.
    -> list of [ntok][rows_i] (llamd_fwd_matvec_tokens; gemm=True: llamd_fwd_gemm_tokens)."""
    x = _f32(x)
    ntok, k = x.shape
    ws = list(weights)
    if not 1 <= len(ws) <= 3 or any(w.blocks() * QK_K != k for w in ws):
        raise ShapeError("matvec_tokens: 1..3 matrices with k columns")
    nb = k // QK_K
    dx, dq, dd = DevBuf.from_array(x), DevBuf(ntok * k), DevBuf(ntok * nb * 4)
    lib().llamd_fwd_quantize(dx.ptr, dq.ptr, dd.ptr, ntok * nb)
    outs = [DevBuf(ntok * w.rows() * 4) for w in ws]
    wp = [w.ptr for w in ws] + [None] * (3 - len(ws))
    op = [o.ptr for o in outs] + [None] * (3 - len(ws))
    rows = [w.rows() for w in ws] + [0] * (3 - len(ws))
    if gemm == "tc":  # tolerance-level tcgen05 path
        d16 = DevBuf(ntok * k * 4)  # two f16 terms per element
        lib().llamd_fwd_act_f16_rm(dq.ptr, dd.ptr, d16.ptr, ntok * nb)
        lib().llamd_fwd_gemm_tokens_tc(wp[0], wp[1], wp[2], d16.ptr, op[0], op[1], op[2], nb, rows[0], rows[1], rows[2], ntok)
        _tc_check()
    elif gemm:
        drm = DevBuf(ntok * k)
        lib().llamd_fwd_q8k_residue_major(dq.ptr, drm.ptr, ntok * nb)
        lib().llamd_fwd_gemm_tokens(wp[0], wp[1], wp[2], drm.ptr, dd.ptr, op[0], op[1], op[2], nb, rows[0], rows[1], rows[2], ntok)
    else:
        lib().llamd_fwd_matvec_tokens(wp[0], wp[1], wp[2], dq.ptr, dd.ptr, op[0], op[1], op[2], nb, rows[0], rows[1], rows[2], ntok)
    backend.sync()
    return [o.download_f32(ntok * w.rows()).reshape(ntok, w.rows()) for o, w in zip(outs, ws)]


def expert_major(weights, x, ids, rows_per_expert: int, by_slot: bool = False, gemm=False):
    """Routed matvec for many tokens through the scatter plan.

    `weights`: 1-2 DeviceWeights holding n_expert matrices of rows_per_expert
    rows; ids int32 [ntok][n_used]. by_slot=False: x is [ntok][k] and pair
    (t, s) reads x[t] (gate/up); by_slot=True: x is [ntok*n_used][k] and pair p
    reads x[p] (down). -> list of [ntok*n_used][rows_per_expert], row block p =
    expert ids[p] applied to its activation."""
    x = _f32(x)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    ntok, n_used = ids.shape
    ws = list(weights)
    k = x.shape[1]
    if not 1 <= len(ws) <= 2 or any(w.blocks() * QK_K != k or w.rows() % rows_per_expert for w in ws):
        raise ShapeError("expert_major: 1..2 expert tensors with k columns")
    n_expert = ws[0].rows() // rows_per_expert
    if ids.size and (ids.min() < 0 or ids.max() >= n_expert):
        raise Malformed(f"expert id outside 0..{n_expert}")
    if x.shape[0] != (ntok * n_used if by_slot else ntok):
        raise ShapeError("expert_major: activation rows")
    nb, npair, nact = k // QK_K, ntok * n_used, x.shape[0]
    dx, dq, dd = DevBuf.from_array(x), DevBuf(nact * k), DevBuf(nact * nb * 4)
    lib().llamd_fwd_quantize(dx.ptr, dq.ptr, dd.ptr, nact * nb)
    di = DevBuf.from_array(ids)
    gs, gc, pt, ps = DevBuf(n_expert * 4), DevBuf(n_expert * 4), DevBuf(npair * 4), DevBuf(npair * 4)
    max_items = npair // 8 + n_expert
    wk, nw = DevBuf((max_items + 1) * 12), DevBuf.zeroed(4)
    lib().llamd_fwd_moe_group_work(di.ptr, n_expert, n_used, ntok, gs.ptr, gc.ptr, pt.ptr, ps.ptr, wk.ptr, nw.ptr)
    outs = [DevBuf.zeroed(npair * rows_per_expert * 4) for _ in ws]
    if gemm == "tc":  # tolerance-level tcgen05 path
        d16 = DevBuf(nact * k * 4)
        lib().llamd_fwd_act_f16_rm(dq.ptr, dd.ptr, d16.ptr, nact * nb)
        lib().llamd_fwd_expert_gemm_tc(ws[0].ptr, ws[1].ptr if len(ws) > 1 else None, gs.ptr, gc.ptr, ps.ptr if by_slot else pt.ptr, ps.ptr,
                                       d16.ptr, outs[0].ptr, outs[1].ptr if len(ws) > 1 else None, nb, rows_per_expert, n_expert, npair)
        _tc_check()
    elif gemm:
        drm = DevBuf(nact * k)
        lib().llamd_fwd_q8k_residue_major(dq.ptr, drm.ptr, nact * nb)
        lib().llamd_fwd_expert_gemm(ws[0].ptr, ws[1].ptr if len(ws) > 1 else None, gs.ptr, gc.ptr, ps.ptr if by_slot else pt.ptr, ps.ptr,
                                    drm.ptr, dd.ptr, outs[0].ptr, outs[1].ptr if len(ws) > 1 else None, nb, rows_per_expert, n_expert)
    else:
        lib().llamd_fwd_expert_major(ws[0].ptr, ws[1].ptr if len(ws) > 1 else None, wk.ptr, nw.ptr, max_items, ps.ptr if by_slot else pt.ptr,
                                     ps.ptr, dq.ptr, dd.ptr, outs[0].ptr, outs[1].ptr if len(ws) > 1 else None, nb, rows_per_expert, n_expert)
    backend.sync()
    return [o.download_f32(npair * rows_per_expert).reshape(npair, rows_per_expert) for o in outs]


def matvec_f32act(w: "backend.DeviceWeights", x):
    """f32 activations [nseq][k]; quantized inside the matvec (llamd_fwd_matvec_f32act)."""
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    if x2.shape[1] != w.blocks() * QK_K or not 1 <= x2.shape[0] <= backend.MAX_SEQ:
        raise ShapeError("matvec_f32act sizes")
    dx, do = DevBuf.from_array(x2), DevBuf(x2.shape[0] * w.rows() * 4)
    lib().llamd_fwd_matvec_f32act(w.ptr, dx.ptr, do.ptr, w.blocks(), w.rows(), x2.shape[0])
    backend.sync()
    return do.download_f32(x2.shape[0] * w.rows()).reshape(x2.shape[0], w.rows())


def matvec_grouped_pa_silu(w: "backend.DeviceWeights", ids, gate, up, rows_per_expert: int):
    """Down projection of routed experts with silu(gate)*up and its quantization fused in.
    ids int32 [n_slots]; gate/up f32 [n_slots][k] -> [n_slots][rows_per_expert]."""
    gate, up = _f32(gate), _f32(up)
    ids = np.ascontiguousarray(ids, dtype=np.int32).ravel()
    if gate.shape != up.shape or gate.shape[0] != ids.size or gate.shape[1] != w.blocks() * QK_K or w.rows() % rows_per_expert:
        raise ShapeError("matvec_grouped_pa_silu sizes")
    n_expert = w.rows() // rows_per_expert
    if ids.size == 0 or ids.min() < 0 or ids.max() >= n_expert:
        raise Malformed(f"expert id outside 0..{n_expert}")
    dg, du, di, do = DevBuf.from_array(gate), DevBuf.from_array(up), DevBuf.from_array(ids), DevBuf(ids.size * rows_per_expert * 4)
    lib().llamd_fwd_matvec_grouped_pa_silu(w.ptr, di.ptr, dg.ptr, du.ptr, do.ptr, w.blocks(), rows_per_expert, ids.size, 1)
    backend.sync()
    return do.download_f32(ids.size * rows_per_expert).reshape(ids.size, rows_per_expert)


def matvec_grouped_pa(w: "backend.DeviceWeights", ids, qs, d, rows_per_expert: int):
    """Down projection of routed experts, every slot with its own Q8_K activation (op::planar_grouped_per_act).
    ids int32 [n_slots]; qs int8 [n_slots][k]; d f32 [n_slots][k/256] -> [n_slots][rows_per_expert]."""
    ids = np.ascontiguousarray(ids, dtype=np.int32).ravel()
    qs = np.ascontiguousarray(qs, dtype=np.int8).reshape(ids.size, -1)
    d = _f32(d).reshape(ids.size, -1)
    if qs.shape[1] != w.blocks() * QK_K or d.shape[1] != w.blocks() or w.rows() % rows_per_expert:
        raise ShapeError("matvec_grouped_pa sizes")
    n_expert = w.rows() // rows_per_expert
    if ids.size == 0 or ids.min() < 0 or ids.max() >= n_expert:
        raise Malformed(f"expert id outside 0..{n_expert}")
    dq, dd, di, do = DevBuf.from_array(qs), DevBuf.from_array(d), DevBuf.from_array(ids), DevBuf(ids.size * rows_per_expert * 4)
    lib().llamd_fwd_matvec_grouped_pa_batch(w.ptr, di.ptr, dq.ptr, dd.ptr, do.ptr, w.blocks(), rows_per_expert, ids.size, 1)
    backend.sync()
    return do.download_f32(ids.size * rows_per_expert).reshape(ids.size, rows_per_expert)


def matvec_grouped_x2_silu_quant(wa: "backend.DeviceWeights", wb: "backend.DeviceWeights", ids, x, rows_per_expert: int, fused: bool = True):
    """gate/up of routed experts for nseq sequences, then act = silu(gate)*up as Q8_K.
    ids int32 [nseq][n_used]; x f32 [nseq][k]. fused=True: one launch (llamd_fwd_matvec_grouped_x2_silu_quant);
    False: the two separate launches. -> (gate, up, qs int8 [slots][rows], d f32 [slots][rows/256])."""
    x = _f32(x)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    nseq, n_used = ids.shape
    k = x.shape[1]
    if x.shape[0] != nseq or wa.blocks() * QK_K != k or wb.blocks() != wa.blocks() or rows_per_expert % QK_K:
        raise ShapeError("matvec_grouped_x2_silu_quant sizes")
    n_expert = wa.rows() // rows_per_expert
    if ids.min() < 0 or ids.max() >= n_expert:
        raise Malformed(f"expert id outside 0..{n_expert}")
    nb, slots = k // QK_K, nseq * n_used
    dx, dq, dd = DevBuf.from_array(x), DevBuf(nseq * k), DevBuf(nseq * nb * 4)
    lib().llamd_fwd_quantize(dx.ptr, dq.ptr, dd.ptr, nseq * nb)
    di = DevBuf.from_array(ids)
    dg, du = DevBuf(slots * rows_per_expert * 4), DevBuf(slots * rows_per_expert * 4)
    q2, d2 = DevBuf(slots * rows_per_expert), DevBuf(slots * (rows_per_expert // QK_K) * 4)
    if fused:
        dc = DevBuf.zeroed(slots * 4)
        lib().llamd_fwd_matvec_grouped_x2_silu_quant(wa.ptr, wb.ptr, di.ptr, dq.ptr, dd.ptr, dg.ptr, du.ptr, dc.ptr, q2.ptr, d2.ptr, nb,
                                                     rows_per_expert, n_used, nseq)
        backend.sync()
        assert not dc.download(np.uint32, slots).any(), "arrival counters must return to zero"
    else:
        lib().llamd_fwd_matvec_grouped_x2_batch(wa.ptr, wb.ptr, di.ptr, dq.ptr, dd.ptr, dg.ptr, du.ptr, nb, rows_per_expert, n_used, nseq)
        lib().llamd_fwd_silu_mul_quant(dg.ptr, du.ptr, None, q2.ptr, d2.ptr, slots * rows_per_expert)
        backend.sync()
    return (dg.download_f32(slots * rows_per_expert).reshape(slots, -1), du.download_f32(slots * rows_per_expert).reshape(slots, -1),
            q2.download(np.int8, slots * rows_per_expert).reshape(slots, -1), d2.download_f32(slots * (rows_per_expert // QK_K)).reshape(slots, -1))


def attention_meta_quant(q, k, v, positions, n_head: int, n_head_kv: int, hd: int, max_kv: int, fused: bool = True):
    """nseq sequences, each with its own cache k/v [nseq][max_kv][n_head_kv*hd] and position; the attention output and
    its Q8_K form. fused=True: llamd_fwd_attention_meta_quant; False: attention_meta then quantize."""
    q, k, v = _f32(q).ravel(), _f32(k).ravel(), _f32(v).ravel()
    positions = np.ascontiguousarray(positions, dtype=np.int32).ravel()
    nseq, n = positions.size, n_head * hd
    if q.size != nseq * n or k.size != nseq * max_kv * n_head_kv * hd or v.size != k.size or n % QK_K:
        raise ShapeError("attention_meta_quant sizes")
    meta = np.zeros((nseq, 2), dtype=np.int32)
    meta[:, 1] = positions
    dq, dk, dv, do = DevBuf.from_array(q), DevBuf.from_array(k), DevBuf.from_array(v), DevBuf(q.nbytes)
    dm, ds = DevBuf.from_array(meta), DevBuf(nseq * n_head * max_kv * 4)
    qs, d = DevBuf(nseq * n), DevBuf(nseq * (n // QK_K) * 4)
    if fused:
        dc = DevBuf.zeroed(nseq * 4)
        lib().llamd_fwd_attention_meta_quant(dq.ptr, dk.ptr, dv.ptr, do.ptr, ds.ptr, n_head, n_head_kv, hd, dm.ptr, max_kv, nseq, dc.ptr, qs.ptr,
                                             d.ptr)
        backend.sync()
        assert not dc.download(np.uint32, nseq).any(), "arrival counters must return to zero"
    else:
        lib().llamd_fwd_attention_meta(dq.ptr, dk.ptr, dv.ptr, do.ptr, ds.ptr, n_head, n_head_kv, hd, dm.ptr, max_kv, nseq)
        lib().llamd_fwd_quantize(do.ptr, qs.ptr, d.ptr, nseq * (n // QK_K))
        backend.sync()
    return do.download_f32(nseq * n).reshape(nseq, n), qs.download(np.int8, nseq * n).reshape(nseq, n), d.download_f32(nseq * (n // QK_K)).reshape(nseq, -1)
