"""`llamd_tensor::Backend` on the device: the outermost of the reference's three backend surfaces.

``Shape`` and ``Tensor`` follow crates/llamd-tensor/src/{shape.rs:16-117, lib.rs:24-117} (ggml order: ``dims[0]`` is the
contiguous axis, a "row" is ``dims[0]`` elements, at most 4 dims, no zero dim). ``CudaBackend`` has the trait's ten
methods (crates/llamd-tensor/src/lib.rs:148-174) with `&Tensor` in and an owned `Tensor` out; each runs one kernel of
csrc/backend_ops.cu with CpuBackend's arithmetic (crates/llamd-cpu/src/lib.rs:55-225) and refuses what CpuBackend
refuses, with the same error kinds, before any device call. Host tensors go to the device and back on every call:
this surface is the reference's unfused, checkable form of each op (`forward_layer` calls it as `&dyn Backend`);
the resident model (``model.CudaModel``) is the fast path and computes the same values.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from . import backend
from ._lib import lib
from .backend import DevBuf, Malformed, ShapeError

MAX_DIMS = 4


class Shape:
    def __init__(self, dims):
        dims = [int(d) for d in dims]
        if not 1 <= len(dims) <= MAX_DIMS:
            raise Malformed(f"shape: rank {len(dims)} is outside 1..={MAX_DIMS}")
        if 0 in dims:
            raise Malformed(f"shape: {dims} has a zero dimension")
        self._dims = tuple(dims)

    @classmethod
    def from_gguf(cls, dims):
        return cls(dims)

    def rank(self):
        return len(self._dims)

    def dims(self):
        return list(self._dims)

    def dim(self, i):
        return self._dims[i] if i < len(self._dims) else 1

    def elems(self):
        return math.prod(self._dims)

    def row_len(self):
        return self._dims[0]

    def rows(self):
        return math.prod(self._dims[1:])

    def strides(self):
        s, acc = [0] * MAX_DIMS, 1
        for i, d in enumerate(self._dims):
            s[i] = acc
            acc *= d
        return s

    def offset(self, idx):
        if len(idx) != len(self._dims) or any(c >= d for c, d in zip(idx, self._dims)):
            return None
        return sum(c * s for c, s in zip(idx, self.strides()))

    def same_as(self, other: "Shape"):
        if self._dims != other._dims:
            raise ShapeError(f"shape mismatch: expected {self.dims()}, got {other.dims()}")

    def __eq__(self, o):
        return isinstance(o, Shape) and self._dims == o._dims

    def __hash__(self):
        return hash(self._dims)

    def __repr__(self):
        return str(list(self._dims))


class Tensor:
    def __init__(self, shape: Shape, data):
        data = np.ascontiguousarray(data, dtype=np.float32).ravel()
        if data.size != shape.elems():
            raise Malformed(f"tensor: shape {shape} needs {shape.elems()} elements, got {data.size}")
        self._shape, self._data = shape, data

    @classmethod
    def zeros(cls, shape: Shape):
        return cls(shape, np.zeros(shape.elems(), np.float32))

    @classmethod
    def from_slice(cls, dims, data):
        return cls(Shape(dims), data)

    def shape(self):
        return self._shape

    def data(self):
        return self._data

    def elems(self):
        return self._data.size

    def rows(self):
        return self._shape.rows()

    def row_len(self):
        return self._shape.row_len()

    def row(self, i):
        n = self.row_len()
        return self._data[i * n:(i + 1) * n] if 0 <= i < self.rows() else None

    def reshape(self, dims):
        s = Shape(dims)
        if s.elems() != self._data.size:
            raise Malformed(f"reshape: {self._data.size} elements cannot become {s}")
        return Tensor(s, self._data.copy())


class RopeConfig:
    """crates/llamd-tensor/src/lib.rs:126-142."""

    def __init__(self, head_dim: int, freq_base: float, freq_scale: float = 1.0):
        self.head_dim, self.freq_base, self.freq_scale = int(head_dim), np.float32(freq_base), np.float32(freq_scale)


def rope_sincos(positions, cfg: RopeConfig) -> np.ndarray:
    """[len(positions)][head_dim/2][2] = (sin, cos) of theta = pos*freq_scale / freq_base^(2i/d), every step in f32
    and with the host libm, as crates/llamd-cpu/src/lib.rs:184-201 computes them (Rust's powf / sin_cos call the
    platform libm). One row per distinct position is computed, then gathered."""
    d, half = cfg.head_dim, cfg.head_dim // 2
    libm = C.CDLL("libm.so.6")
    for f, n in ((libm.powf, 2), (libm.sinf, 1), (libm.cosf, 1)):
        f.restype, f.argtypes = C.c_float, [C.c_float] * n
    i = np.arange(half, dtype=np.float32)
    exponent = np.float32(2.0) * i / np.float32(d)
    denom = np.array([libm.powf(float(cfg.freq_base), float(e)) for e in exponent], dtype=np.float32)
    pos = np.asarray(positions, dtype=np.uint32)
    uniq, inverse = np.unique(pos, return_inverse=True)
    tab = np.empty((uniq.size, half, 2), np.float32)
    for r, p in enumerate(uniq):
        theta = (np.float32(p) * cfg.freq_scale) / denom
        tab[r, :, 0] = [libm.sinf(float(t)) for t in theta]
        tab[r, :, 1] = [libm.cosf(float(t)) for t in theta]
    return np.ascontiguousarray(tab[inverse])


class CudaBackend:
    """impl Backend for the CUDA device. No CPU fallback: without a device every method raises Unsupported."""

    def __init__(self):
        if not backend.available():
            raise backend.Unsupported("cuda: no device present (there is no CPU fallback)")
        backend.stream_init()
        self._L = lib()

    def name(self) -> str:
        return "cuda-b200"

    # -- helpers ---------------------------------------------------------------
    def _run(self, shape: Shape, fn, *inputs) -> Tensor:
        bufs = [DevBuf.from_array(a) for a in inputs]
        out = DevBuf(shape.elems() * 4)
        fn(out, *bufs)
        backend.sync()
        return Tensor(shape, out.download_f32(shape.elems()))

    def _zip(self, a: Tensor, b: Tensor, f) -> Tensor:
        a.shape().same_as(b.shape())
        return self._run(a.shape(), lambda o, da, db: f(da.ptr, db.ptr, o.ptr, a.elems()), a.data(), b.data())

    # -- the trait ---------------------------------------------------------------
    def rms_norm(self, x: Tensor, eps: float) -> Tensor:
        return self._run(x.shape(), lambda o, dx: self._L.llamd_fwd_rms_norm_rows(dx.ptr, o.ptr, x.row_len(), x.rows(), C.c_float(eps)), x.data())

    def softmax(self, x: Tensor) -> Tensor:
        return self._run(x.shape(), lambda o, dx: self._L.llamd_fwd_softmax_rows(dx.ptr, o.ptr, x.row_len(), x.rows()), x.data())

    def silu(self, x: Tensor) -> Tensor:
        return self._run(x.shape(), lambda o, dx: self._L.llamd_fwd_silu(dx.ptr, o.ptr, x.elems()), x.data())

    def add(self, a: Tensor, b: Tensor) -> Tensor:
        if a.elems() >= 2**31:
            raise backend.Unsupported("add: more than 2^31 elements")
        return self._zip(a, b, self._L.llamd_fwd_add)

    def mul(self, a: Tensor, b: Tensor) -> Tensor:
        return self._zip(a, b, self._L.llamd_fwd_mul)

    def scale(self, x: Tensor, by: float) -> Tensor:
        return self._run(x.shape(), lambda o, dx: self._L.llamd_fwd_scale(dx.ptr, C.c_float(by), o.ptr, x.elems()), x.data())

    def matmul(self, w: Tensor, x: Tensor) -> Tensor:
        """w [k, m], x [k, n] -> [m, n]: a dot product over rows, both operands sharing the contiguous axis k."""
        k = w.row_len()
        if x.row_len() != k:
            raise ShapeError(f"shape mismatch: expected {[k]}, got {[x.row_len()]}")
        m, n = w.rows(), x.rows()
        return self._run(Shape([m, n]), lambda o, dw, dx: self._L.llamd_fwd_matmul_f32(dw.ptr, dx.ptr, o.ptr, k, m, n), w.data(), x.data())

    def rope(self, x: Tensor, positions, cfg: RopeConfig) -> Tensor:
        d = cfg.head_dim
        if d % 2:
            raise Malformed(f"rope: head_dim {d} must be even")
        if x.row_len() % d:
            raise Malformed(f"rope: row length {x.row_len()} is not a multiple of head_dim {d}")
        positions = list(positions)
        if len(positions) != x.rows():
            raise Malformed(f"rope: {len(positions)} positions for {x.rows()} rows")
        sc = rope_sincos(positions, cfg)
        return self._run(x.shape(), lambda o, dx, ds: self._L.llamd_fwd_rope_rows(dx.ptr, o.ptr, x.row_len(), x.rows(), d, ds.ptr), x.data(), sc)

    def get_rows(self, table: Tensor, ids) -> Tensor:
        ids = [int(i) for i in ids]
        for i in ids:
            if not 0 <= i < table.rows():
                raise Malformed(f"get_rows: id {i} is outside a table of {table.rows()} rows")
        n = table.row_len()
        shape = Shape([n, len(ids)])  # refuses an empty id list, as Shape::new does
        return self._run(shape, lambda o, dt, di: self._L.llamd_fwd_get_rows_f32(dt.ptr, di.ptr, o.ptr, n, len(ids)), table.data(),
                         np.asarray(ids, dtype=np.uint32))
