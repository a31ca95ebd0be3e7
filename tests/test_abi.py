"""CPU-side checks of the drop-in boundary: the shared library loads without a
GPU, exports every symbol the headers declare, and the wrappers refuse bad
arguments before any FFI call (the reference's own stub-build test,
crates/llamd-rocm/src/lib.rs:933-955)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    import __graft_entry__ as g

    g.build()
    from llamd_rs_b200 import _lib

    return _lib


def declared_symbols(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(llamd_(?:cuda|fwd|model|gguf)_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built):
    L = C.CDLL(built.SO)
    names = declared_symbols("llamd_cuda.h") + declared_symbols("llamd_cuda_model.h") + declared_symbols("llamd_gguf.h")
    assert len(names) > 80
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, f"declared but not exported: {missing}"


def test_python_binding_covers_the_header(built):
    bound = set(built.SIGNATURES)
    declared = set(declared_symbols("llamd_cuda.h"))
    assert declared <= bound, f"unbound: {sorted(declared - bound)}"
    built.lib()  # resolves every bound symbol or raises
    from llamd_rs_b200 import gguf

    assert set(declared_symbols("llamd_gguf.h")) <= set(gguf.SIGNATURES)
    gguf._bind()


def test_headers_cite_the_reference_and_compile_as_c(built, tmp_path):
    for h in ("llamd_cuda.h", "llamd_cuda_model.h", "llamd_gguf.h"):
        text = open(os.path.join(ROOT, "include", h)).read()
        assert "crates/llamd-r" in text, "each header cites the reference interface it replaces"
    src = tmp_path / "t.c"
    src.write_text('#include "llamd_cuda.h"\n#include "llamd_cuda_model.h"\n#include "llamd_gguf.h"\nint main(void){return LLAMD_T_FFN_DOWN_EXPS==14?0:1;}\n')
    import subprocess

    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(tmp_path / "t")])
    subprocess.check_call([str(tmp_path / "t")])


def test_availability_is_reported_not_assumed(built):
    from llamd_rs_b200 import backend

    n = backend.device_count()
    assert n >= 0 and backend.available() == (n > 0)
    assert backend.built_with_cuda()


def test_bad_arguments_are_refused_before_the_ffi(built):
    from llamd_rs_b200 import backend

    with pytest.raises(backend.Malformed):
        backend.matvec_q6k(np.zeros(0, np.uint8), [], [], 0)
    with pytest.raises(backend.Malformed):
        backend.DeviceWeights.upload(np.zeros(10, np.uint8), 1, 1)  # short weights
    with pytest.raises(backend.Malformed):
        backend.quantize_q8k_on_device(np.zeros(100, np.float32))
    with pytest.raises(backend.Malformed):
        backend.device_info(backend.device_count())
    dw = backend.DeviceWeights(None, 8, 2)  # handle without a device: only the host-side checks run
    with pytest.raises(backend.ShapeError):
        dw.matvec(np.zeros(256, np.int8), np.zeros(1, np.float32))
    for bad in ([], [-1], [2]):
        with pytest.raises(backend.Malformed):
            dw.matvec_grouped(np.zeros(512, np.int8), np.zeros(2, np.float32), bad, 4)
    with pytest.raises(backend.Malformed):
        dw.matvec_grouped(np.zeros(512, np.int8), np.zeros(2, np.float32), [0], 3)  # non-divisor


def test_no_device_means_an_error_not_a_fallback(built):
    from llamd_rs_b200 import backend
    from llamd_rs_b200.model import CudaModel
    from llamd_rs_b200 import synth

    if backend.available():
        pytest.skip("a device is present")
    with pytest.raises(backend.Unsupported):
        backend.DeviceWeights.upload(np.zeros(210, np.uint8), 1, 1)
    with pytest.raises(backend.Unsupported):
        CudaModel(synth.TINY, 16)
    with pytest.raises(backend.Unsupported):
        backend.stream_init()


def test_product_never_imports_the_oracle():
    """Only tests/, smoke() and the bench's CPU legs may touch oracle/."""
    pkg = os.path.join(ROOT, "llamd_rs_b200")
    offenders = []
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                if re.search(r"^\s*(import|from)\s+oracle\b", text, flags=re.M) or "llamd_oracle" in text:
                    offenders.append(f)
    assert not offenders, offenders
