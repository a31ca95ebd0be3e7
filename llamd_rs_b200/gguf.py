"""GGUF files: the reader in libllamd_cuda.so seen from Python, and a writer.

``Gguf`` mirrors the reference's type of that name (crates/llamd-gguf/src/lib.rs:104-286): ``open`` / ``parse``,
``get``, ``architecture``, ``tensor``, ``tensor_data``; ``hparams`` and ``verify_present`` are
``Hparams::from_gguf`` (crates/llamd-models/src/hparams.rs:78-149) and ``Model::verify_present``
(crates/llamd-models/src/model.rs:133-160). Errors carry the reference's kinds (``backend.Malformed``,
``backend.Unsupported``, ``OSError`` for I/O).

``write_gguf`` writes version 3 files from numpy arrays. The tests use it to put the synthetic models into a file;
it also lets the random-init benchmark model be handed to the reference itself, which only loads GGUF.
"""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np

from . import _lib, backend

E_OK, E_MALFORMED, E_UNSUPPORTED, E_IO, E_OTHER, E_ABSENT = 0, -1, -2, -3, -4, -5
GGML_F32, GGML_F16, GGML_Q8_0, GGML_Q6_K = 0, 1, 8, 14

_ERR_LEN = 512
_bound = None


def _bind():
    global _bound
    if _bound is not None:
        return _bound
    L = _lib.lib()
    vp, i32, u64, sz, cp = C.c_void_p, C.c_int, C.c_uint64, C.c_size_t, C.c_char_p
    sig = {
        "llamd_gguf_open": (vp, [cp, C.POINTER(i32), cp, sz]),
        "llamd_gguf_parse": (vp, [vp, sz, C.POINTER(i32), cp, sz]),
        "llamd_gguf_close": (None, [vp]),
        "llamd_gguf_version": (C.c_uint32, [vp]),
        "llamd_gguf_alignment": (u64, [vp]),
        "llamd_gguf_data_offset": (u64, [vp]),
        "llamd_gguf_file_size": (u64, [vp]),
        "llamd_gguf_n_metadata": (u64, [vp]),
        "llamd_gguf_n_tensors": (u64, [vp]),
        "llamd_gguf_get_u64": (i32, [vp, cp, C.POINTER(u64)]),
        "llamd_gguf_get_f32": (i32, [vp, cp, C.POINTER(C.c_float)]),
        "llamd_gguf_get_str": (i32, [vp, cp, cp, sz, C.POINTER(sz)]),
        "llamd_gguf_get_array_len": (i32, [vp, cp, C.POINTER(u64)]),
        "llamd_gguf_metadata_key": (cp, [vp, u64]),
        "llamd_gguf_find_tensor": (C.c_int64, [vp, cp]),
        "llamd_gguf_tensor_name": (cp, [vp, u64]),
        "llamd_gguf_tensor_info": (i32, [vp, u64, C.POINTER(C.c_uint32), C.POINTER(i32), C.POINTER(u64), C.POINTER(u64)]),
        "llamd_gguf_tensor_data": (i32, [vp, u64, C.POINTER(vp), C.POINTER(sz), cp, sz]),
        "llamd_gguf_hparams": (i32, [vp, vp, C.POINTER(i32), C.POINTER(C.c_int32), C.POINTER(C.c_int32), cp, sz]),
        "llamd_gguf_verify_present": (i32, [vp, cp, sz]),
        "llamd_model_load_gguf": (vp, [vp, i32, i32, C.POINTER(i32), cp, sz]),
    }
    for name, (res, args) in sig.items():
        f = getattr(L, name)
        f.restype, f.argtypes = res, args
    _bound = L
    return L


SIGNATURES = (
    "llamd_gguf_open llamd_gguf_parse llamd_gguf_close llamd_gguf_version llamd_gguf_alignment llamd_gguf_data_offset "
    "llamd_gguf_file_size llamd_gguf_n_metadata llamd_gguf_n_tensors llamd_gguf_get_u64 llamd_gguf_get_f32 llamd_gguf_get_str "
    "llamd_gguf_get_array_len llamd_gguf_metadata_key llamd_gguf_find_tensor llamd_gguf_tensor_name llamd_gguf_tensor_info "
    "llamd_gguf_tensor_data llamd_gguf_hparams llamd_gguf_verify_present llamd_model_load_gguf"
).split()


def raise_kind(kind: int, msg: str):
    if kind == E_MALFORMED:
        raise backend.Malformed(msg)
    if kind == E_UNSUPPORTED:
        raise backend.Unsupported(msg)
    if kind == E_IO:
        raise OSError(msg)
    raise backend.Other(msg)


class TensorInfo:
    """TensorInfo (lib.rs:88-102)."""

    def __init__(self, index, name, dims, ggml_type, offset):
        self.index, self.name, self.dims, self.ggml_type, self.offset = index, name, dims, ggml_type, offset

    def elems(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    def __repr__(self):
        return f"TensorInfo({self.name!r}, dims={self.dims}, type={self.ggml_type}, offset={self.offset})"


class Gguf:
    def __init__(self, handle, keep=None):
        self._L = _bind()
        self._h = handle
        self._keep = keep  # bytes a parse() handle points into

    @classmethod
    def open(cls, path) -> "Gguf":
        L = _bind()
        kind, err = C.c_int(0), C.create_string_buffer(_ERR_LEN)
        h = L.llamd_gguf_open(str(path).encode(), C.byref(kind), err, _ERR_LEN)
        if not h:
            raise_kind(kind.value, err.value.decode(errors="replace"))
        return cls(h)

    @classmethod
    def parse(cls, data: bytes) -> "Gguf":
        L = _bind()
        buf = np.frombuffer(bytes(data), dtype=np.uint8) if len(data) else np.zeros(1, np.uint8)
        kind, err = C.c_int(0), C.create_string_buffer(_ERR_LEN)
        h = L.llamd_gguf_parse(buf.ctypes.data_as(C.c_void_p), len(data), C.byref(kind), err, _ERR_LEN)
        if not h:
            raise_kind(kind.value, err.value.decode(errors="replace"))
        return cls(h, keep=buf)

    def close(self):
        if self._h:
            self._L.llamd_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # -- header --------------------------------------------------------------
    version = property(lambda s: s._L.llamd_gguf_version(s._h))
    alignment = property(lambda s: s._L.llamd_gguf_alignment(s._h))
    data_offset = property(lambda s: s._L.llamd_gguf_data_offset(s._h))

    def file_size(self) -> int:
        return self._L.llamd_gguf_file_size(self._h)

    # -- metadata ------------------------------------------------------------
    def keys(self):
        return [self._L.llamd_gguf_metadata_key(self._h, i).decode(errors="replace") for i in range(self._L.llamd_gguf_n_metadata(self._h))]

    def get_u64(self, key: str):
        v = C.c_uint64()
        return v.value if self._L.llamd_gguf_get_u64(self._h, key.encode(), C.byref(v)) == E_OK else None

    def get_f32(self, key: str):
        v = C.c_float()
        return v.value if self._L.llamd_gguf_get_f32(self._h, key.encode(), C.byref(v)) == E_OK else None

    def get_str(self, key: str):
        n = C.c_size_t()
        if self._L.llamd_gguf_get_str(self._h, key.encode(), None, 0, C.byref(n)) != E_OK:
            return None
        out = C.create_string_buffer(n.value + 1)
        self._L.llamd_gguf_get_str(self._h, key.encode(), out, n.value + 1, None)
        return out.raw[: n.value].decode(errors="replace")

    def get_array_len(self, key: str):
        v = C.c_uint64()
        return v.value if self._L.llamd_gguf_get_array_len(self._h, key.encode(), C.byref(v)) == E_OK else None

    def architecture(self):
        return self.get_str("general.architecture")

    # -- tensors -------------------------------------------------------------
    def _info(self, i: int) -> TensorInfo:
        ty, nd, off = C.c_uint32(), C.c_int(), C.c_uint64()
        dims = (C.c_uint64 * 4)()
        self._L.llamd_gguf_tensor_info(self._h, i, C.byref(ty), C.byref(nd), dims, C.byref(off))
        name = self._L.llamd_gguf_tensor_name(self._h, i).decode(errors="replace")
        return TensorInfo(i, name, [int(dims[d]) for d in range(nd.value)], ty.value, off.value)

    @property
    def tensors(self):
        return [self._info(i) for i in range(self._L.llamd_gguf_n_tensors(self._h))]

    def tensor(self, name: str):
        i = self._L.llamd_gguf_find_tensor(self._h, name.encode())
        return None if i < 0 else self._info(i)

    def tensor_data(self, t: TensorInfo) -> np.ndarray:
        """The tensor's bytes inside the mapping (a view: valid until close)."""
        p, n, err = C.c_void_p(), C.c_size_t(), C.create_string_buffer(_ERR_LEN)
        rc = self._L.llamd_gguf_tensor_data(self._h, t.index, C.byref(p), C.byref(n), err, _ERR_LEN)
        if rc != E_OK:
            raise_kind(rc, err.value.decode(errors="replace"))
        if n.value == 0:
            return np.zeros(0, np.uint8)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(n.value,))

    # -- model level ---------------------------------------------------------
    def hparams(self) -> dict:
        from .model import _Hparams

        h, moe, n_ff, n_ctx = _Hparams(), C.c_int(), C.c_int32(), C.c_int32()
        err = C.create_string_buffer(_ERR_LEN)
        rc = self._L.llamd_gguf_hparams(self._h, C.byref(h), C.byref(moe), C.byref(n_ff), C.byref(n_ctx), err, _ERR_LEN)
        if rc != E_OK:
            raise_kind(rc, err.value.decode(errors="replace"))
        out = {k: getattr(h, k) for k, _ in _Hparams._fields_}
        out.update(arch="qwen3moe" if moe.value else "qwen3", n_ff=n_ff.value, n_ctx_train=n_ctx.value)
        return out

    def verify_present(self) -> None:
        err = C.create_string_buffer(_ERR_LEN)
        rc = self._L.llamd_gguf_verify_present(self._h, err, _ERR_LEN)
        if rc != E_OK:
            raise_kind(rc, err.value.decode(errors="replace"))


# ---- writer -------------------------------------------------------------------------------------------------------
_BLOCK = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_Q8_0: (32, 34), GGML_Q6_K: (256, 210)}
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}


class Typed:
    """A metadata value with an explicit GGUF type id (0 U8 ... 12 F64; 9 = array, then ``inner`` is the element type)."""

    def __init__(self, ty: int, value, inner: int | None = None):
        self.ty, self.value, self.inner = ty, value, inner


def _gstr(s) -> bytes:
    b = s if isinstance(s, bytes) else str(s).encode()
    return struct.pack("<Q", len(b)) + b


def _infer(v) -> int:
    if isinstance(v, bool):
        return 7
    if isinstance(v, (int, np.integer)):
        return 4 if 0 <= int(v) < 2**32 else (10 if int(v) >= 0 else 11)
    if isinstance(v, (float, np.floating)):
        return 6
    if isinstance(v, (str, bytes)):
        return 8
    if isinstance(v, (list, tuple)):
        return 9
    raise TypeError(f"no GGUF type for {type(v).__name__}")


def _value(ty: int, v, inner: int | None = None) -> bytes:
    if ty == 8:
        return _gstr(v)
    if ty == 9:  # a plain list: its first item decides the element type
        inner = inner if inner is not None else (_infer(v[0]) if len(v) else 4)
        return struct.pack("<IQ", inner, len(v)) + b"".join(_value(inner, x) for x in v)
    return struct.pack(_SCALAR[ty], v)


def tensor_nbytes(ggml_type: int, dims) -> int:
    n = 1
    for d in dims:
        n *= int(d)
    be, bb = _BLOCK[ggml_type]
    if n % be:
        raise backend.Malformed(f"tensor length: {n} elements is not a multiple of the {be}-element block")
    return n // be * bb


def write_gguf(path, metadata: dict, tensors, alignment: int = 32) -> int:
    """Write a version-3 file. ``metadata`` maps key -> value (type inferred: int U32/U64/I64, float F32, str, bool,
    list) or key -> ``Typed``. ``tensors`` is a list of (name, dims, ggml_type, data) with ``dims`` in
    ggml order (fastest first: a [rows x k] matrix is [k, rows]) and ``data`` an array or a zero-argument callable
    yielding arrays, so that a tensor larger than memory can be produced piece by piece. Returns the file size."""
    meta = dict(metadata)
    if alignment != 32 and "general.alignment" not in meta:
        meta["general.alignment"] = Typed(4, alignment)
    head = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(meta)))
    for k, v in meta.items():
        t = v if isinstance(v, Typed) else Typed(_infer(v), v)
        head += _gstr(k) + struct.pack("<I", t.ty) + _value(t.ty, t.value, t.inner)
    offsets, off = [], 0
    for name, dims, ty, _ in tensors:
        offsets.append(off)
        nb = tensor_nbytes(ty, dims)
        off += (nb + alignment - 1) // alignment * alignment
    for (name, dims, ty, _), o in zip(tensors, offsets):
        head += _gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", int(d)) for d in dims) + struct.pack("<IQ", ty, o)
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        for (name, dims, ty, data), o in zip(tensors, offsets):
            want, wrote = tensor_nbytes(ty, dims), 0
            for piece in (data() if callable(data) else (data,)):
                b = np.ascontiguousarray(piece).view(np.uint8).ravel()
                f.write(b.data)
                wrote += b.size
            if wrote != want:
                raise backend.Malformed(f"{name}: {wrote} bytes given, dims and type want {want}")
            f.write(b"\0" * ((-want) % alignment))
        return f.tell()


def synthetic_metadata(hp: dict) -> dict:
    """The metadata keys Hparams::from_gguf reads (hparams.rs:78-149), for a qwen3moe model of these sizes."""
    p = "qwen3moe"
    return {
        "general.architecture": p,
        "general.name": "synthetic",
        f"{p}.block_count": hp["n_layer"],
        f"{p}.context_length": 262144,
        f"{p}.embedding_length": hp["n_embd"],
        f"{p}.feed_forward_length": 5472,
        f"{p}.attention.head_count": hp["n_head"],
        f"{p}.attention.head_count_kv": hp["n_head_kv"],
        f"{p}.attention.key_length": hp["head_dim"],
        f"{p}.attention.value_length": hp["head_dim"],
        f"{p}.rope.freq_base": float(hp["rope_freq_base"]),
        f"{p}.attention.layer_norm_rms_epsilon": float(hp["rms_eps"]),
        f"{p}.expert_count": hp["n_expert"],
        f"{p}.expert_used_count": hp["n_expert_used"],
        f"{p}.expert_feed_forward_length": hp["n_ff_expert"],
    }


def write_synthetic(path, hp: dict, seed: int) -> int:
    """The random-init model of ``CudaModel.load_synthetic(hp, seed, ...)`` as a GGUF file, byte for byte the same
    tensors, generated expert by expert so that the full-size model (23.4 GiB) needs no more memory than one expert."""
    from . import synth

    E, V, ne, ffe = hp["n_embd"], hp["n_vocab"], hp["n_expert"], hp["n_ff_expert"]
    qd, kvd = hp["n_head"] * hp["head_dim"], hp["n_head_kv"] * hp["head_dim"]
    ts = [
        ("token_embd.weight", [E, V], GGML_Q6_K, lambda: iter([synth.q6k_blocks(V * E // 256, seed, "tok_embd")])),
        ("output_norm.weight", [E], GGML_F32, np.ones(E, np.float32)),
        ("output.weight", [E, V], GGML_Q6_K, lambda: iter([synth.q6k_blocks(V * E // 256, seed, "output")])),
    ]
    names = {"attn_norm": ("attn_norm.weight", [E], GGML_F32), "attn_q": ("attn_q.weight", [E, qd], GGML_Q6_K),
             "attn_k": ("attn_k.weight", [E, kvd], GGML_Q6_K), "attn_v": ("attn_v.weight", [E, kvd], GGML_Q6_K),
             "attn_q_norm": ("attn_q_norm.weight", [hp["head_dim"]], GGML_F32), "attn_k_norm": ("attn_k_norm.weight", [hp["head_dim"]], GGML_F32),
             "attn_out": ("attn_output.weight", [qd, E], GGML_Q6_K), "ffn_norm": ("ffn_norm.weight", [E], GGML_F32),
             "ffn_gate_inp": ("ffn_gate_inp.weight", [E, ne], GGML_F32)}
    for il in range(hp["n_layer"]):
        def lay(key, il=il):  # regenerated when written: nothing of a layer is held while the others are listed
            return lambda: iter([synth.layer_weights(hp, seed, il, with_experts=False)[key]])
        for key, (suffix, dims, ty) in names.items():
            ts.append((f"blk.{il}.{suffix}", dims, ty, lay(key)))
        for which, (suffix, dims) in enumerate([("ffn_gate_exps.weight", [E, ffe, ne]), ("ffn_up_exps.weight", [E, ffe, ne]), ("ffn_down_exps.weight", [ffe, E, ne])]):
            def experts(il=il, which=which):
                return (synth.expert_blocks(hp, seed, il, which, e) for e in range(ne))
            ts.append((f"blk.{il}.{suffix}", dims, GGML_Q6_K, experts))
    return write_gguf(path, synthetic_metadata(hp), ts)
