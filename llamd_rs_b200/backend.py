"""Python mirror of the reference's device-backend crate surface, over the C ABI.

Same names, argument meaning and error behaviour as ``llamd-rocm``
(crates/llamd-rocm/src/lib.rs, crates/llamd-rocm/src/forward.rs): every
wrapper validates lengths and ids BEFORE the FFI call, device buffers free on
drop, host-facing calls synchronise. numpy arrays stand in for Rust slices.
This module is for tests, the bench and Python users; the compiled host side
(stream, graph, scratch, the resident model) is C++ inside the library.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from ._lib import lib

QK_K = 256
Q6K_BLOCK_BYTES = 210
Q8_0_BLOCK_BYTES = 34
MAX_SEQ = 8
MAX_BATCH = 256  # LLAMD_MAX_BATCH: sequences a model can hold (beyond MAX_SEQ a pass runs on the prefill GEMM kernels)


class LlamdError(RuntimeError):
    """Base of the errors below (llamd_core::Error, crates/llamd-core/src/lib.rs:18-43)."""


class ShapeError(LlamdError):
    pass


class Malformed(LlamdError):
    pass


class Unsupported(LlamdError):
    pass


class Other(LlamdError):
    pass


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _last_error() -> str:
    return lib().llamd_cuda_last_error_string().decode(errors="replace")


def built_with_cuda() -> bool:
    try:
        lib()
        return True
    except Exception:
        return False


def device_count() -> int:
    return int(lib().llamd_cuda_device_count())


def available() -> bool:
    return device_count() > 0


def _need_device():
    if not available():
        raise Unsupported("cuda: no device present (there is no CPU fallback)")


@dataclass
class DeviceInfo:
    index: int
    name: str
    total_mem: int
    free_mem: int
    sm_count: int
    warp_size: int
    arch: str


def device_info(index: int) -> DeviceInfo:
    n = device_count()
    if index < 0 or index >= n:
        raise Malformed(f"cuda device: index {index} of {n} devices")
    name = C.create_string_buffer(256)
    arch = C.create_string_buffer(64)
    total, sms, warp = C.c_size_t(0), C.c_int(0), C.c_int(0)
    rc = lib().llamd_cuda_device_info(index, name, 256, arch, 64, C.byref(total), C.byref(sms), C.byref(warp))
    if rc != 0:
        raise Other(f"cudaGetDeviceProperties failed for device {index}")
    return DeviceInfo(index, name.value.decode(), total.value, int(lib().llamd_cuda_free_mem()), sms.value, warp.value,
                      arch.value.decode())


def set_device(index: int) -> None:
    n = device_count()
    if index < 0 or index >= n:
        raise Malformed(f"cuda device: index {index} of {n} devices")
    if lib().llamd_cuda_set_device(index) != 0:
        raise Other("set_device: " + _last_error())


def free_memory() -> int:
    return int(lib().llamd_fwd_free_mem())


def stream_init() -> None:
    _need_device()
    if lib().llamd_fwd_stream_init() != 0:
        raise Other("stream creation failed: " + _last_error())


def sync() -> None:
    """Stream sync + sticky error check (crates/llamd-rocm/src/forward.rs:240-260)."""
    rc = lib().llamd_fwd_sync()
    if rc != 0:
        msg = _last_error()
        lib().llamd_fwd_last_error()
        raise Other("device error: " + msg)


def check() -> None:
    """Raise if a launch recorded an argument error (no synchronise)."""
    e = lib().llamd_fwd_last_error()
    if e != 0:
        raise Other(f"device error {e}: " + _last_error())


class DevBuf:
    """Owned device allocation (crates/llamd-rocm/src/forward.rs:29-218)."""

    def __init__(self, nbytes: int):
        _need_device()
        self.nbytes = int(nbytes)
        self.ptr = lib().llamd_fwd_alloc(self.nbytes)
        if not self.ptr:
            raise Other(f"cudaMalloc failed for {nbytes} bytes: " + _last_error())

    @classmethod
    def zeroed(cls, nbytes: int) -> "DevBuf":
        b = cls(nbytes)
        b.zero()
        return b

    @classmethod
    def from_array(cls, a) -> "DevBuf":
        a = np.ascontiguousarray(a)
        b = cls(max(a.nbytes, 1))
        b.upload(a)
        return b

    from_bytes = from_array
    from_f32 = from_array

    def upload(self, a) -> None:
        a = np.ascontiguousarray(a)
        if a.nbytes > self.nbytes:
            raise ShapeError(f"upload of {a.nbytes} bytes into a buffer of {self.nbytes}")
        if lib().llamd_fwd_upload(self.ptr, _ptr(a), a.nbytes) != 0:
            raise Other("upload failed: " + _last_error())
        sync()  # the host array may be freed by the caller right after

    upload_bytes = upload_i32 = upload

    def download(self, dtype, count: int) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        if out.nbytes > self.nbytes:
            raise ShapeError(f"download of {out.nbytes} bytes from a buffer of {self.nbytes}")
        if lib().llamd_fwd_download(_ptr(out), self.ptr, out.nbytes) != 0:
            raise Other("download failed: " + _last_error())
        return out

    def download_f32(self, count: int) -> np.ndarray:
        return self.download(np.float32, count)

    def download_i32(self, count: int) -> np.ndarray:
        return self.download(np.int32, count)

    def zero(self) -> None:
        lib().llamd_fwd_memset(self.ptr, 0, self.nbytes)

    def bytes(self) -> int:
        return self.nbytes

    def free(self) -> None:
        if getattr(self, "ptr", None):
            lib().llamd_fwd_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _split_act(qs, d, blocks: int, nact: int = 1):
    qs = np.ascontiguousarray(qs, dtype=np.int8).ravel()
    d = np.ascontiguousarray(d, dtype=np.float32).ravel()
    if d.size != blocks * nact or qs.size != blocks * nact * QK_K:
        raise ShapeError(f"expected {blocks * nact} activation blocks, got {d.size}")
    return qs, d


class DeviceWeights:
    """Q6_K weights resident on the device (crates/llamd-rocm/src/lib.rs:259-362).

    ``w`` is the reference's packed 210-byte blocks, ``rows`` x ``blocks``; the
    upload permutes them into the tiled device layout.
    """

    def __init__(self, ptr, rows: int, blocks: int):
        self.ptr, self._rows, self._blocks = ptr, rows, blocks

    @classmethod
    def upload(cls, w, rows: int, blocks: int) -> "DeviceWeights":
        w = np.ascontiguousarray(w, dtype=np.uint8).ravel()
        need = rows * blocks * Q6K_BLOCK_BYTES
        if rows <= 0 or blocks <= 0 or w.size < need:
            raise Malformed(f"device weights: need {need} bytes for {rows}x{blocks}, have {w.size}")
        _need_device()
        ptr = lib().llamd_cuda_upload_q6k(_ptr(w), rows * blocks)
        if not ptr:
            raise Other("cudaMalloc/cudaMemcpy failed for weights: " + _last_error())
        return cls(ptr, rows, blocks)

    def rows(self) -> int:
        return self._rows

    def blocks(self) -> int:
        return self._blocks

    def matvec(self, qs, d) -> np.ndarray:
        qs, d = _split_act(qs, d, self._blocks)
        out = np.zeros(self._rows, dtype=np.float32)
        rc = lib().llamd_cuda_matvec_q6k_resident(self.ptr, _ptr(qs), _ptr(d), _ptr(out), self._blocks, self._rows)
        if rc != 0:
            raise Other("CUDA resident matvec failed: " + _last_error())
        return out

    def matvec_f32(self, x, nseq: int = 1) -> np.ndarray:
        """Model::matvec_quant for nseq f32 activations: quantize on device, then matvec."""
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        if nseq < 1 or nseq > MAX_SEQ or x.size != nseq * self._blocks * QK_K:
            raise ShapeError(f"expected {nseq}x{self._blocks * QK_K} activations, got {x.size}")
        out = np.zeros(nseq * self._rows, dtype=np.float32)
        rc = lib().llamd_cuda_matvec_q6k_f32(self.ptr, _ptr(x), _ptr(out), self._blocks, self._rows, nseq)
        if rc != 0:
            raise Other("CUDA matvec failed: " + _last_error())
        return out.reshape(nseq, self._rows)

    def _check_grouped(self, expert_ids, rows_per_expert: int):
        ids = np.ascontiguousarray(expert_ids, dtype=np.int32).ravel()
        if ids.size == 0:
            raise Malformed("expert_ids: empty")
        if rows_per_expert <= 0 or self._rows % rows_per_expert != 0:
            raise Malformed(f"rows_per_expert: {rows_per_expert} does not divide {self._rows} uploaded rows")
        n_expert = self._rows // rows_per_expert
        bad = ids[(ids < 0) | (ids >= n_expert)]
        if bad.size:
            raise Malformed(f"expert id: {int(bad[0])} outside 0..{n_expert}")
        return ids

    def matvec_grouped(self, qs, d, expert_ids, rows_per_expert: int) -> np.ndarray:
        """[n_used][rows_per_expert], unscaled (crates/llamd-rocm/src/lib.rs:434-508)."""
        qs, d = _split_act(qs, d, self._blocks)
        ids = self._check_grouped(expert_ids, rows_per_expert)
        out = np.zeros(rows_per_expert * ids.size, dtype=np.float32)
        rc = lib().llamd_cuda_matvec_grouped(self.ptr, _ptr(ids), _ptr(qs), _ptr(d), _ptr(out), self._blocks,
                                             rows_per_expert, ids.size)
        if rc != 0:
            raise Other("CUDA grouped matvec failed: " + _last_error())
        return out.reshape(ids.size, rows_per_expert)

    def bench_kernel_only(self, qs, d, iters: int) -> float:
        qs, d = _split_act(qs, d, self._blocks)
        if iters == 0:
            raise Malformed("bench iters: 0")
        ms = C.c_float(0)
        rc = lib().llamd_cuda_matvec_bench(self.ptr, _ptr(qs), _ptr(d), self._blocks, self._rows, iters, C.byref(ms))
        if rc != 0:
            raise Other("CUDA kernel-only bench failed: " + _last_error())
        return float(ms.value)

    def bench_grouped_kernel_only(self, qs, d, expert_ids, rows_per_expert: int, iters: int) -> float:
        if iters == 0:
            raise Malformed("grouped bench args: invalid")
        qs, d = _split_act(qs, d, self._blocks)
        ids = self._check_grouped(expert_ids, rows_per_expert)
        ms = C.c_float(0)
        rc = lib().llamd_cuda_matvec_grouped_bench(self.ptr, _ptr(ids), _ptr(qs), _ptr(d), self._blocks, rows_per_expert,
                                                   ids.size, iters, C.byref(ms))
        if rc != 0:
            raise Other("CUDA grouped bench failed: " + _last_error())
        return float(ms.value)

    def unpack(self) -> np.ndarray:
        """The reference-layout bytes recovered from the tiled device buffer."""
        n = self._rows * self._blocks
        tmp = DevBuf(n * Q6K_BLOCK_BYTES)
        lib().llamd_fwd_unpack_q6k(self.ptr, tmp.ptr, n)
        return tmp.download(np.uint8, n * Q6K_BLOCK_BYTES)

    def dequantize(self, first_block: int = 0, n_blocks: int | None = None) -> np.ndarray:
        n = self._rows * self._blocks
        if n_blocks is None:
            n_blocks = n - first_block
        if first_block < 0 or n_blocks < 0 or first_block + n_blocks > n:
            raise Malformed(f"dequantize: blocks {first_block}+{n_blocks} of {n}")
        tmp = DevBuf(max(n_blocks, 1) * QK_K * 4)
        lib().llamd_fwd_dequantize_q6k(self.ptr, first_block, n_blocks, tmp.ptr)
        return tmp.download_f32(n_blocks * QK_K)

    def free(self):
        if getattr(self, "ptr", None):
            lib().llamd_cuda_release(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Q80Weights:
    """Q8_0 weights on the device; matvec is dequantize-then-f32-dot in the
    reference's order (crates/llamd-models/src/model.rs:253-263)."""

    def __init__(self, ptr, rows, blocks32):
        self.ptr, self._rows, self._blocks = ptr, rows, blocks32

    @classmethod
    def upload(cls, w, rows: int, blocks32: int) -> "Q80Weights":
        w = np.ascontiguousarray(w, dtype=np.uint8).ravel()
        need = rows * blocks32 * Q8_0_BLOCK_BYTES
        if rows <= 0 or blocks32 <= 0 or w.size < need:
            raise Malformed(f"device weights: need {need} bytes for {rows}x{blocks32}, have {w.size}")
        _need_device()
        ptr = lib().llamd_cuda_upload_q8_0(_ptr(w), rows, blocks32)
        if not ptr:
            raise Other("upload failed: " + _last_error())
        return cls(ptr, rows, blocks32)

    def matvec_f32(self, x, nseq: int = 1) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        if nseq < 1 or nseq > MAX_SEQ or x.size != nseq * self._blocks * 32:
            raise ShapeError(f"expected {nseq}x{self._blocks * 32} activations, got {x.size}")
        out = np.zeros(nseq * self._rows, dtype=np.float32)
        rc = lib().llamd_cuda_matvec_q8_0_f32(self.ptr, _ptr(x), _ptr(out), self._blocks, self._rows, nseq)
        if rc != 0:
            raise Other("CUDA Q8_0 matvec failed: " + _last_error())
        return out.reshape(nseq, self._rows)

    def dequantize(self) -> np.ndarray:
        tmp = DevBuf(self._rows * self._blocks * 32 * 4)
        lib().llamd_fwd_dequantize_q8_0(self.ptr, self._rows, self._blocks, tmp.ptr)
        return tmp.download_f32(self._rows * self._blocks * 32).reshape(self._rows, self._blocks * 32)

    def free(self):
        if getattr(self, "ptr", None):
            lib().llamd_cuda_release(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def quantize_q8k_on_device(x):
    """-> (qs int8[n], d f32[nb], bsums int16[nb*16]) (crates/llamd-rocm/src/lib.rs:569-617)."""
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    if x.size == 0 or x.size % QK_K != 0:
        raise Malformed(f"q8k input: {x.size} is not a multiple of {QK_K}")
    _need_device()
    nb = x.size // QK_K
    qs = np.zeros(x.size, dtype=np.int8)
    d = np.zeros(nb, dtype=np.float32)
    bs = np.zeros(nb * 16, dtype=np.int16)
    rc = lib().llamd_cuda_quantize_q8k(_ptr(x), nb, _ptr(qs), _ptr(d), _ptr(bs))
    if rc != 0:
        raise Other("CUDA q8_k quantize failed: " + _last_error())
    return qs, d, bs


def matvec_q6k(w, qs, d, rows: int) -> np.ndarray:
    """Upload-per-call convenience (crates/llamd-rocm/src/lib.rs:914-927)."""
    d = np.ascontiguousarray(d, dtype=np.float32).ravel()
    if d.size == 0 or rows == 0:
        raise Malformed(f"cuda matvec: {rows} rows, {d.size} blocks")
    dw = DeviceWeights.upload(w, rows, d.size)
    try:
        return dw.matvec(qs, d)
    finally:
        dw.free()
