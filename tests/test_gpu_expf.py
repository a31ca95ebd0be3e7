"""The device's exponential against the host libm's expf, bit for bit.

The reference's softmax, SiLU, router and attention call Rust's f32::exp, i.e. the platform libm's expf, which is
not correctly rounded everywhere. The library corrects its own (correctly rounded) exponential to it with a table
built by comparing EVERY float input when the stream is made; here that equality is checked through the elementwise
entry point on dense runs of consecutive bit patterns, on random inputs and at the ends of the range, and through
the composite ops (softmax, SiLU) that the tolerance-level tests used to bound within an ulp.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from llamd_rs_b200 import backend

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    backend.stream_init()
    return backend


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_exception_table_exists(be):
    from llamd_rs_b200._lib import lib

    n = lib().llamd_cuda_exp_exceptions()
    # glibc's expf differs from the correctly rounded value on a few inputs in 100000; none at all would mean the
    # comparison did not run, millions would mean the two functions are not the same function
    assert 100 < n < 5_000_000, n
    # the cheap test that spares most inputs the look-up: a window around rounding midpoints, measured over every listed
    # input at start-up; well under a hundredth of an ulp for glibc's expf
    assert 0 < lib().llamd_cuda_exp_window_on() < (1 << 22)


@pytest.mark.parametrize("first", [0x33000000, 0x3F000000, 0x3F800000, 0x40A00000, 0x42AF0000, 0xB3000000, 0xBE000000, 0xC0000000, 0xC1F00000, 0xC2C00000])
def test_dense_runs_of_consecutive_floats(be, orc, first):
    from llamd_rs_b200 import ops

    x = (np.uint32(first) + np.arange(1 << 21, dtype=np.uint32)).view(np.float32)
    got, want = ops.expf(x), orc.expf(x)
    bad = np.flatnonzero(bits(got) != bits(want))
    assert bad.size == 0, f"{bad.size} of {x.size} differ, first x={x[bad[0]]!r}: gpu {got[bad[0]]!r} host {want[bad[0]]!r}"


def test_random_inputs_and_the_ends_of_the_range(be, orc):
    from llamd_rs_b200 import ops

    rng = np.random.default_rng(7)
    x = np.concatenate([
        rng.uniform(-104.0, 89.0, 1 << 22).astype(np.float32),
        rng.standard_normal(1 << 22).astype(np.float32) * np.float32(8.0),
        np.array([0.0, -0.0, 1e-30, -1e-30, 2.0 ** -25, -(2.0 ** -25), 2.0 ** -26, 88.72283, 88.72284, 89.0, 100.0, np.inf,
                  -87.3, -103.9, -103.98, -104.0, -104.5, -150.0, -np.inf], np.float32),
    ])
    got, want = ops.expf(x), orc.expf(x)
    bad = np.flatnonzero(bits(got) != bits(want))
    assert bad.size == 0, f"{bad.size} differ, first x={x[bad[0]]!r}: gpu {got[bad[0]]!r} host {want[bad[0]]!r}"


def test_softmax_and_silu_are_bit_identical_to_the_cpu_ops(be, orc):
    from llamd_rs_b200 import ops, synth
    from llamd_rs_b200.tensor_backend import CudaBackend, Tensor

    cb = CudaBackend()
    x = synth.normal_f32(64 * 1000, 9, "expf.softmax").reshape(64, 1000) * np.float32(3.0)
    got = cb.softmax(Tensor.from_slice([1000, 64], x.ravel())).data().reshape(64, 1000)  # ggml order: ne[0] = row length
    assert np.array_equal(bits(got), bits(orc.softmax(x)))
    v = synth.normal_f32(1 << 20, 9, "expf.silu") * np.float32(6.0)
    ones = np.ones_like(v)
    assert np.array_equal(bits(ops.silu_mul(v, ones)), bits(orc.mul(orc.silu(v), ones)))
    assert np.array_equal(bits(cb.silu(Tensor.from_slice([v.size], v)).data()), bits(orc.silu(v)))
