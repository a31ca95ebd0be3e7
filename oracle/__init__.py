"""ctypes binding of the CPU oracle (``llamd_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the CPU-baseline legs of ``bench.py``. Nothing under the shipped package
imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libllamd_oracle.so")

F32, F16, Q8_0, Q6K = 0, 1, 8, 14
QK_K = 256
Q6K_BLOCK_BYTES = 210
Q8_0_BLOCK_BYTES = 34


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile if it is stale."""
    src = os.path.join(_HERE, "llamd_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_bytes_for.restype = C.c_int64
        L.orc_bytes_for.argtypes = [C.c_int, C.c_int64]
        L.orc_nearest_int.restype = C.c_int
        L.orc_nearest_int.argtypes = [C.c_float]
        L.orc_dot_q6k_q8k.restype = C.c_float
        L.orc_argmax.restype = C.c_int32
        L.orc_argmax.argtypes = [C.c_void_p, C.c_int64]
        L.orc_kv_new.restype = C.c_void_p
        L.orc_kv_new.argtypes = [C.c_int, C.c_int, C.c_int]
        L.orc_kv_free.argtypes = [C.c_void_p]
        L.orc_kv_set_f16.argtypes = [C.c_void_p, C.c_int]
        L.orc_round_to_f16.restype = C.c_float
        L.orc_round_to_f16.argtypes = [C.c_float]
        L.orc_kv_keys.restype = C.c_void_p
        L.orc_kv_keys.argtypes = [C.c_void_p, C.c_int]
        L.orc_kv_values.restype = C.c_void_p
        L.orc_kv_values.argtypes = [C.c_void_p, C.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


# ---------------------------------------------------------------- formats
def f16_to_f32(bits: int) -> float:
    return float(lib().orc_f16_to_f32(bits))


def f32_to_f16(v: float) -> int:
    return int(lib().orc_f32_to_f16(C.c_float(v)))


def bytes_for(ty: int, n: int) -> int:
    return int(lib().orc_bytes_for(ty, n))


def dequantize(ty: int, src, n: int) -> np.ndarray:
    src = _u8(src)
    out = np.zeros(max(n, 0), dtype=np.float32)
    rc = lib().orc_dequantize(C.c_int(ty), _p(src), C.c_int64(src.size), C.c_int64(n), _p(out))
    if rc != 0:
        raise ValueError(f"orc_dequantize refused: {rc}")
    return out


def nearest_int(v: float) -> int:
    return int(lib().orc_nearest_int(C.c_float(v)))


def quantize_q8k(x):
    """-> (qs int8 [n], d f32 [nb], bsums int16 [nb*16])"""
    x = _f32(x).ravel()
    assert x.size % QK_K == 0
    nb = x.size // QK_K
    qs = np.zeros(x.size, dtype=np.int8)
    d = np.zeros(nb, dtype=np.float32)
    bs = np.zeros(nb * 16, dtype=np.int16)
    lib().orc_quantize_q8k(_p(x), C.c_int(nb), _p(qs), _p(d), _p(bs))
    return qs, d, bs


def dot_q6k_q8k(w, qs, d, n: int) -> float:
    w = _u8(w)
    qs = np.ascontiguousarray(qs, dtype=np.int8)
    d = _f32(d)
    return float(lib().orc_dot_q6k_q8k(_p(w), _p(qs), _p(d), C.c_int(n)))


def matvec_q6k_q8k(w, qs, d, k: int, rows: int, threads: int = 1) -> np.ndarray:
    w = _u8(w)
    qs = np.ascontiguousarray(qs, dtype=np.int8)
    d = _f32(d)
    y = np.zeros(rows, dtype=np.float32)
    lib().orc_matvec_q6k_q8k(_p(w), _p(qs), _p(d), C.c_int(k), C.c_int64(rows), _p(y), C.c_int(threads))
    return y


def matvec_q6k(w, x, k: int, rows: int, threads: int = 1) -> np.ndarray:
    w = _u8(w)
    x = _f32(x)
    y = np.zeros(rows, dtype=np.float32)
    rc = lib().orc_matvec_q6k(_p(w), _p(x), C.c_int(k), C.c_int64(rows), _p(y), C.c_int(threads))
    if rc:
        raise ValueError(rc)
    return y


def matvec_dequant(ty: int, w, x, k: int, rows: int, threads: int = 1) -> np.ndarray:
    w = np.ascontiguousarray(w)
    x = _f32(x)
    y = np.zeros(rows, dtype=np.float32)
    rc = lib().orc_matvec_dequant(C.c_int(ty), _p(w), _p(x), C.c_int(k), C.c_int64(rows), _p(y), C.c_int(threads))
    if rc:
        raise ValueError(rc)
    return y


def repack_q6k_planar(src, rows: int, blocks: int):
    src = _u8(src)
    off = (C.c_int64 * 5)()
    rc = lib().orc_repack_q6k_planar(_p(src), C.c_int64(src.size), C.c_int64(rows), C.c_int64(blocks), None, off)
    if rc:
        raise ValueError("short source")
    out = np.zeros(off[4], dtype=np.uint8)
    lib().orc_repack_q6k_planar(_p(src), C.c_int64(src.size), C.c_int64(rows), C.c_int64(blocks), _p(out), off)
    return out, list(off)


# ---------------------------------------------------------------- cpu ops
def rms_norm(x, eps: float) -> np.ndarray:
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    out = np.zeros_like(x2)
    lib().orc_rms_norm(_p(x2), C.c_int(x2.shape[1]), C.c_int(x2.shape[0]), C.c_float(eps), _p(out))
    return out.reshape(x.shape)


def softmax(x) -> np.ndarray:
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    out = np.zeros_like(x2)
    lib().orc_softmax(_p(x2), C.c_int(x2.shape[1]), C.c_int(x2.shape[0]), _p(out))
    return out.reshape(x.shape)


def silu(x) -> np.ndarray:
    x = _f32(x)
    out = np.zeros_like(x)
    lib().orc_silu(_p(x), C.c_int64(x.size), _p(out))
    return out


def expf(x) -> np.ndarray:
    """The host libm's expf, elementwise (what Rust's f32::exp lowers to)."""
    x = _f32(x).ravel()
    out = np.zeros_like(x)
    lib().orc_expf(_p(x), C.c_int64(x.size), _p(out))
    return out


def add(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.zeros_like(a)
    lib().orc_add(_p(a), _p(b), C.c_int64(a.size), _p(out))
    return out


def mul(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.zeros_like(a)
    lib().orc_mul(_p(a), _p(b), C.c_int64(a.size), _p(out))
    return out


def scale(x, by: float) -> np.ndarray:
    x = _f32(x)
    out = np.zeros_like(x)
    lib().orc_scale(_p(x), C.c_float(by), C.c_int64(x.size), _p(out))
    return out


def matmul(w, x) -> np.ndarray:
    """w [m rows of k], x [n rows of k] -> [n, m] (reference layout out[j*m+i])."""
    w, x = _f32(w), _f32(x)
    m, k = w.shape
    n = x.shape[0]
    out = np.zeros((n, m), dtype=np.float32)
    lib().orc_matmul(_p(w), _p(x), C.c_int(k), C.c_int(m), C.c_int(n), _p(out))
    return out


def rope(x, positions, head_dim: int, freq_base: float, freq_scale: float = 1.0) -> np.ndarray:
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    pos = np.ascontiguousarray(positions, dtype=np.uint32)
    assert pos.size == x2.shape[0]
    out = np.zeros_like(x2)
    rc = lib().orc_rope(_p(x2), C.c_int(x2.shape[1]), C.c_int(x2.shape[0]), _p(pos), C.c_int(head_dim),
                        C.c_float(freq_base), C.c_float(freq_scale), _p(out))
    if rc:
        raise ValueError("rope refused")
    return out.reshape(x.shape)


def rope_angles(pos: int, head_dim: int, freq_base: float, freq_scale: float = 1.0):
    s = np.zeros(head_dim // 2, dtype=np.float32)
    c = np.zeros(head_dim // 2, dtype=np.float32)
    lib().orc_rope_angles(C.c_uint32(pos), C.c_int(head_dim), C.c_float(freq_base), C.c_float(freq_scale), _p(s), _p(c))
    return s, c


def get_rows(table, ids) -> np.ndarray:
    table = _f32(table)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    out = np.zeros((ids.size, table.shape[1]), dtype=np.float32)
    rc = lib().orc_get_rows(_p(table), C.c_int(table.shape[1]), C.c_int(table.shape[0]), _p(ids), C.c_int(ids.size), _p(out))
    if rc:
        raise ValueError("id outside the table")
    return out


def route(logits, n_used: int):
    """-> dict(experts int32[n_used], weights_raw, weight_sum, weights, probs)"""
    logits = _f32(logits)
    n = logits.size
    ex = np.zeros(max(n_used, 1), dtype=np.int32)
    wr = np.zeros(max(n_used, 1), dtype=np.float32)
    w = np.zeros(max(n_used, 1), dtype=np.float32)
    ws = C.c_float(0)
    probs = np.zeros(n, dtype=np.float32)
    rc = lib().orc_route(_p(logits), C.c_int(n), C.c_int(n_used), _p(ex), _p(wr), C.byref(ws), _p(w), _p(probs))
    if rc:
        raise ValueError("impossible routing request")
    return dict(experts=ex[:n_used], weights_raw=wr[:n_used], weight_sum=float(ws.value), weights=w[:n_used], probs=probs)


def attend(q, k, v, n_kv: int, n_head: int, n_head_kv: int, head_dim: int) -> np.ndarray:
    q, k, v = _f32(q), _f32(k), _f32(v)
    if q.size != n_head * head_dim or k.size != n_kv * n_head_kv * head_dim or v.size != k.size:
        raise ValueError("shape")
    out = np.zeros(n_head * head_dim, dtype=np.float32)
    rc = lib().orc_attend(_p(q), _p(k), _p(v), C.c_int(n_kv), C.c_int(n_head), C.c_int(n_head_kv), C.c_int(head_dim), _p(out))
    if rc:
        raise ValueError("attend refused")
    return out


def argmax(x) -> int:
    x = _f32(x)
    return int(lib().orc_argmax(_p(x), x.size))


# ---------------------------------------------------------------- model
EXPERT_FN = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int)


class _OrcModel(C.Structure):
    _fields_ = [
        ("n_layer", C.c_int32), ("n_embd", C.c_int32), ("n_head", C.c_int32), ("n_head_kv", C.c_int32),
        ("head_dim", C.c_int32), ("n_expert", C.c_int32), ("n_expert_used", C.c_int32),
        ("n_ff_expert", C.c_int32), ("n_vocab", C.c_int32),
        ("rope_freq_base", C.c_float), ("rms_eps", C.c_float),
        ("tok_embd", C.c_void_p), ("output_norm", C.c_void_p), ("output", C.c_void_p),
        ("attn_norm", C.c_void_p), ("attn_q", C.c_void_p), ("attn_k", C.c_void_p), ("attn_v", C.c_void_p),
        ("attn_q_norm", C.c_void_p), ("attn_k_norm", C.c_void_p), ("attn_out", C.c_void_p),
        ("ffn_norm", C.c_void_p), ("ffn_gate_inp", C.c_void_p),
        ("ffn_gate_exps", C.c_void_p), ("ffn_up_exps", C.c_void_p), ("ffn_down_exps", C.c_void_p),
        ("expert_fn", EXPERT_FN), ("expert_user", C.c_void_p), ("threads", C.c_int32),
    ]


class _OrcTrace(C.Structure):
    _names = ["attn_norm", "q", "k", "v", "q_roped", "k_roped", "attn_out", "kqv_out", "ffn_inp", "ffn_norm",
              "moe_logits", "moe_probs", "experts", "weights", "ffn_out", "x_out"]
    _fields_ = [(n, C.c_void_p) for n in _names]


class Model:
    """The oracle's view of a Qwen3MoE-shaped model held in host arrays.

    ``weights`` is the dict produced by ``llamd_rs_b200.synth.make_model`` (or
    any dict with the same keys): top-level ``tok_embd``, ``output_norm``,
    ``output`` and ``layers`` = list of dicts with the per-layer tensors as
    numpy arrays in the reference's (ggml) byte layout. Expert tensors may be
    left out when ``expert_fn(layer, which, expert) -> np.ndarray`` is given.
    """

    def __init__(self, hp: dict, weights: dict, threads: int = 1, expert_fn=None):
        self.hp = dict(hp)
        self.w = weights
        self._keep = []
        L = hp["n_layer"]

        def ptr_array(key, optional=False):
            arr = (C.c_void_p * L)()
            for i, lay in enumerate(weights["layers"]):
                a = lay.get(key)
                if a is None:
                    if not optional:
                        raise KeyError(key)
                    arr[i] = None
                else:
                    a = np.ascontiguousarray(a)
                    self._keep.append(a)
                    arr[i] = a.ctypes.data
            self._keep.append(arr)
            return C.cast(arr, C.c_void_p)

        m = _OrcModel()
        for k in ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_expert", "n_expert_used",
                  "n_ff_expert", "n_vocab"):
            setattr(m, k, int(hp[k]))
        m.rope_freq_base = float(hp["rope_freq_base"])
        m.rms_eps = float(hp["rms_eps"])
        for k in ("tok_embd", "output_norm", "output"):
            a = weights.get(k)
            if a is not None:
                a = np.ascontiguousarray(a)
                self._keep.append(a)
                setattr(m, k, a.ctypes.data)
        for k in ("attn_norm", "attn_q", "attn_k", "attn_v", "attn_q_norm", "attn_k_norm", "attn_out",
                  "ffn_norm", "ffn_gate_inp"):
            setattr(m, k, ptr_array(k))
        has_experts = all("ffn_gate_exps" in lay for lay in weights["layers"])
        if has_experts:
            for k in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
                setattr(m, k, ptr_array(k))
        if expert_fn is not None:
            cache = self._expert_cache = {}

            def _cb(_user, layer, which, expert):
                key = (layer, which, expert)
                a = cache.get(key)
                if a is None:
                    a = np.ascontiguousarray(expert_fn(layer, which, expert), dtype=np.uint8)
                    if len(cache) > 4096:
                        cache.clear()
                    cache[key] = a
                return a.ctypes.data

            self._cb = EXPERT_FN(_cb)
            m.expert_fn = self._cb
        elif not has_experts:
            raise ValueError("expert tensors or expert_fn required")
        m.threads = threads
        self.m = m
        self.kv = None

    def kv_new(self, capacity: int, f16: bool = False):
        """A fresh cache. f16: every appended K/V value is rounded to binary16 (nearest-even) first."""
        self.kv_free()
        self.kv = lib().orc_kv_new(self.hp["n_layer"], self.hp["n_head_kv"] * self.hp["head_dim"], capacity)
        self.kv_capacity = capacity
        if f16:
            lib().orc_kv_set_f16(self.kv, 1)
        return self.kv

    def expert_cache_clear(self):
        """Forget the expert slices ``expert_fn`` has produced so far (they may be views of large arrays)."""
        c = getattr(self, "_expert_cache", None)
        if c is not None:
            c.clear()

    def kv_fill(self, layer: int, first_pos: int, k, v):
        """Write rows [first_pos, first_pos + n) of one layer's cache (k, v: [n, kv_dim] f32)."""
        kvd = self.hp["n_head_kv"] * self.hp["head_dim"]
        k, v = _f32(k).reshape(-1, kvd), _f32(v).reshape(-1, kvd)
        n = k.shape[0]
        if v.shape[0] != n or first_pos < 0 or first_pos + n > self.kv_capacity:
            raise ValueError("kv_fill outside the cache")
        for fn, src in ((lib().orc_kv_keys, k), (lib().orc_kv_values, v)):
            dst = np.ctypeslib.as_array(C.cast(fn(self.kv, layer), C.POINTER(C.c_float)), shape=(self.kv_capacity * kvd,))
            dst[first_pos * kvd:(first_pos + n) * kvd] = src.ravel()

    def kv_free(self):
        if self.kv:
            lib().orc_kv_free(self.kv)
            self.kv = None

    def __del__(self):
        try:
            self.kv_free()
        except Exception:
            pass

    def kv_layer(self, layer: int, n_pos: int):
        kvd = self.hp["n_head_kv"] * self.hp["head_dim"]
        kp = lib().orc_kv_keys(self.kv, layer)
        vp = lib().orc_kv_values(self.kv, layer)
        k = np.ctypeslib.as_array(C.cast(kp, C.POINTER(C.c_float)), shape=(n_pos * kvd,)).copy()
        v = np.ctypeslib.as_array(C.cast(vp, C.POINTER(C.c_float)), shape=(n_pos * kvd,)).copy()
        return k, v

    def forward(self, token: int, pos: int, want_x: bool = False):
        logits = np.zeros(self.hp["n_vocab"], dtype=np.float32)
        xf = np.zeros(self.hp["n_embd"], dtype=np.float32)
        rc = lib().orc_forward(C.byref(self.m), C.c_uint32(token), C.c_uint32(pos), C.c_void_p(self.kv), _p(logits), _p(xf))
        if rc:
            raise ValueError(f"orc_forward refused: {rc}")
        return (logits, xf) if want_x else logits

    def forward_layer(self, il: int, x, pos: int):
        """-> (x_out, trace dict)"""
        hp = self.hp
        x = _f32(x).copy()
        qd, kvd = hp["n_head"] * hp["head_dim"], hp["n_head_kv"] * hp["head_dim"]
        sizes = dict(attn_norm=hp["n_embd"], q=qd, k=kvd, v=kvd, q_roped=qd, k_roped=kvd, attn_out=qd,
                     kqv_out=hp["n_embd"], ffn_inp=hp["n_embd"], ffn_norm=hp["n_embd"],
                     moe_logits=hp["n_expert"], moe_probs=hp["n_expert"], weights=hp["n_expert_used"],
                     ffn_out=hp["n_embd"], x_out=hp["n_embd"])
        tr = _OrcTrace()
        arrs = {}
        for k, n in sizes.items():
            arrs[k] = np.zeros(n, dtype=np.float32)
            setattr(tr, k, arrs[k].ctypes.data)
        arrs["experts"] = np.zeros(hp["n_expert_used"], dtype=np.int32)
        tr.experts = arrs["experts"].ctypes.data
        rc = lib().orc_forward_layer(C.byref(self.m), C.c_int(il), _p(x), C.c_uint32(pos), C.c_void_p(self.kv), C.byref(tr))
        if rc:
            raise ValueError(f"orc_forward_layer refused: {rc}")
        return x, arrs

    def moe_ffn(self, il: int, x, experts, weights) -> np.ndarray:
        x = _f32(x)
        ex = np.ascontiguousarray(experts, dtype=np.int32)
        w = _f32(weights)
        out = np.zeros(self.hp["n_embd"], dtype=np.float32)
        rc = lib().orc_moe_ffn(C.byref(self.m), C.c_int(il), _p(x), _p(ex), _p(w), C.c_int(ex.size), _p(out))
        if rc:
            raise ValueError("moe_ffn refused")
        return out
