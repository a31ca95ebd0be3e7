"""`CudaBackend` -- the ten methods of `llamd_tensor::Backend` (crates/llamd-tensor/src/lib.rs:148-174) -- against the
oracle's restatement of CpuBackend (crates/llamd-cpu/src/lib.rs:55-225), bit for bit (one ulp after an `exp`), on the reference's own
known-answer vectors (cpu/lib.rs:236-368) and on seeded inputs with ragged, single-row, multi-dimensional and
larger-than-one-chunk shapes; and the refusals CpuBackend makes, with the same error kinds."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cb():
    from llamd_rs_b200 import backend
    from llamd_rs_b200.tensor_backend import CudaBackend

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    return CudaBackend()


@pytest.fixture(scope="module")
def tb():
    from llamd_rs_b200 import tensor_backend

    return tensor_backend


@pytest.fixture(scope="module")
def synth():
    from llamd_rs_b200 import synth

    return synth


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).ravel()


def same(got, want, what):
    assert np.array_equal(bits(got.data()), bits(want)), f"{what}: {np.sum(bits(got.data()) != bits(want))} elements differ in some bit"


def near_after_exp(got, want, what):
    """Results downstream of an `exp`. The reference calls the host libm's expf, which is not correctly rounded on
    every input; the device rounds the double-precision exponential once. The two differ by one ulp on fewer than one
    input in a thousand, so: F32_ULP (crates/llamd-core/src/tolerance.rs) everywhere, and bit-equal on at least 99 %."""
    g, w = np.asarray(got.data(), np.float64), np.asarray(want, np.float64).ravel()
    both_nan = np.isnan(g) & np.isnan(w)
    dev = np.abs(g - w) / np.maximum(np.maximum(np.abs(g), np.abs(w)), 1.0)
    assert np.all(both_nan | (dev <= 1.2e-7) | (g == w)), f"{what}: max deviation {np.nanmax(dev)}"
    equal = (bits(got.data()) == bits(want)) | both_nan  # a NaN's sign and payload are the platform's, not the reference's
    assert np.mean(equal) >= 0.99, f"{what}: only {np.mean(equal):.4f} bit-equal"


SHAPES = [[1], [7], [256], [2049], [5000, 3], [64, 5, 2], [3, 2, 2, 2], [2048, 9]]


def rand(tb, synth, dims, *key, std=1.0):
    n = math.prod(dims)
    return tb.Tensor.from_slice(dims, synth.normal_f32(n, 17, "trait", *key, *dims, std=std))


def rows2d(t):
    return t.data().reshape(t.rows(), t.row_len())


def test_name_and_known_answers(cb, tb):
    assert cb.name() == "cuda-b200"
    out = cb.rms_norm(tb.Tensor.from_slice([2], [3.0, 4.0]), 0.0).data()
    rms = np.sqrt(np.float32(12.5))
    assert abs(out[0] - 3.0 / rms) < 1e-6 and abs(out[1] - 4.0 / rms) < 1e-6
    out = cb.softmax(tb.Tensor.from_slice([3], [1.0, 2.0, 3.0])).data()
    big = cb.softmax(tb.Tensor.from_slice([3], [1000.0, 1001.0, 1002.0])).data()
    assert abs(out.sum(dtype=np.float32) - 1.0) < 1e-6 and np.all(np.isfinite(big)) and np.allclose(out, big, atol=1e-5)
    out = cb.silu(tb.Tensor.from_slice([3], [0.0, 1.0, -1.0])).data()
    assert out[0] == 0.0 and abs(out[1] - 1.0 / (1.0 + math.exp(-1.0))) < 1e-6 and -1.0 < out[2] < 0.0
    w = tb.Tensor.from_slice([2, 3], [1, 2, 3, 4, 5, 6])  # three rows of length 2
    out = cb.matmul(w, tb.Tensor.from_slice([2, 1], [1, 1]))
    assert out.shape().dims() == [3, 1] and out.data().tolist() == [3.0, 7.0, 11.0]
    x = tb.Tensor.from_slice([4, 1], [1, 2, 3, 4])
    assert cb.rope(x, [0], tb.RopeConfig(4, 10000.0)).data().tolist() == [1, 2, 3, 4], "position 0 is the identity"
    out = cb.rope(tb.Tensor.from_slice([4, 1], [1, 0, 0, 0]), [1], tb.RopeConfig(4, 10000.0)).data()
    assert abs(out[0] - math.cos(1.0)) < 1e-5 and abs(out[2] - math.sin(1.0)) < 1e-5 and abs(out[1]) < 1e-5
    table = tb.Tensor.from_slice([2, 3], [1, 2, 3, 4, 5, 6])
    got = cb.get_rows(table, [2, 0])
    assert got.shape().dims() == [2, 2] and got.data().tolist() == [5, 6, 1, 2]


@pytest.mark.parametrize("dims", SHAPES)
def test_row_ops_bit_exact(cb, tb, orc, synth, dims):
    x = rand(tb, synth, dims, "x", std=3.0)
    for eps in (0.0, 1e-6):
        same(cb.rms_norm(x, eps), orc.rms_norm(rows2d(x), eps), f"rms_norm {dims} eps {eps}")
    near_after_exp(cb.softmax(x), orc.softmax(rows2d(x)), f"softmax {dims}")
    near_after_exp(cb.silu(x), orc.silu(x.data()), f"silu {dims}")
    y = rand(tb, synth, dims, "y")
    same(cb.add(x, y), orc.add(x.data(), y.data()), f"add {dims}")
    same(cb.mul(x, y), orc.mul(x.data(), y.data()), f"mul {dims}")
    same(cb.scale(x, 0.3), orc.scale(x.data(), 0.3), f"scale {dims}")
    assert cb.softmax(x).shape() == x.shape()


def test_softmax_and_silu_extremes(cb, tb, orc):
    v = np.array([-1e30, -104.0, -88.0, -20.0, -0.0, 0.0, 1e-30, 20.0, 88.0, 89.0, 1e30, -np.inf], np.float32)
    near_after_exp(cb.silu(tb.Tensor.from_slice([v.size], v)), orc.silu(v), "silu extremes")
    rows = np.stack([v[:8], np.full(8, -50.0, np.float32), np.linspace(-100, 100, 8).astype(np.float32)])
    near_after_exp(cb.softmax(tb.Tensor.from_slice([8, 3], rows)), orc.softmax(rows), "softmax extremes")


@pytest.mark.parametrize("k,m,n", [(1, 1, 1), (2, 3, 1), (7, 5, 3), (32, 32, 8), (33, 40, 9), (2048, 128, 1), (770, 65, 17)])
def test_matmul_bit_exact(cb, tb, orc, synth, k, m, n):
    w = tb.Tensor.from_slice([k, m], synth.normal_f32(k * m, 17, "mm.w", k, m, n, std=0.05))
    x = tb.Tensor.from_slice([k, n], synth.normal_f32(k * n, 17, "mm.x", k, m, n))
    got = cb.matmul(w, x)
    assert got.shape().dims() == [m, n]
    same(got, orc.matmul(rows2d(w), rows2d(x)), f"matmul k={k} m={m} n={n}")


def test_matmul_of_zeros_is_plus_zero(cb, tb):
    """The chain starts from +0.0 (cpu/lib.rs:139), not from the -0.0 an iterator sum starts from."""
    got = cb.matmul(tb.Tensor.from_slice([2, 1], [-0.0, -0.0]), tb.Tensor.from_slice([2, 1], [1.0, 1.0]))
    assert bits(got.data())[0] == 0


@pytest.mark.parametrize("hd,heads,positions,base,scale", [
    (4, 1, [0], 1e4, 1.0), (8, 2, [37, 0, 5], 1e7, 1.0), (128, 4, [511, 512, 4095, 511], 1e7, 1.0), (64, 3, [7, 100000], 1e4, 0.25),
])
def test_rope_bit_exact(cb, tb, orc, synth, hd, heads, positions, base, scale):
    x = tb.Tensor.from_slice([hd * heads, len(positions)], synth.normal_f32(hd * heads * len(positions), 17, "rope", hd, heads))
    got = cb.rope(x, positions, tb.RopeConfig(hd, base, scale))
    same(got, orc.rope(rows2d(x), positions, hd, base, scale), f"rope hd={hd}")


def test_get_rows_bit_exact(cb, tb, orc, synth):
    table = tb.Tensor.from_slice([300, 50], synth.normal_f32(15000, 17, "rows"))
    ids = [49, 0, 0, 17, 49, 3]
    got = cb.get_rows(table, ids)
    assert got.shape().dims() == [300, 6]
    same(got, orc.get_rows(rows2d(table), ids), "get_rows")


def test_refusals_match_cpu_backend(cb, tb):
    from llamd_rs_b200.backend import Malformed, ShapeError

    a, b = tb.Tensor.from_slice([4, 2], np.zeros(8)), tb.Tensor.from_slice([2, 4], np.zeros(8))
    for f in (cb.add, cb.mul):
        with pytest.raises(ShapeError):
            f(a, b)
    with pytest.raises(ShapeError):
        cb.matmul(a, b)  # row lengths 4 and 2
    with pytest.raises(Malformed, match="must be even"):
        cb.rope(tb.Tensor.from_slice([6, 1], np.zeros(6)), [0], tb.RopeConfig(3, 1e4))
    with pytest.raises(Malformed, match="not a multiple"):
        cb.rope(tb.Tensor.from_slice([6, 1], np.zeros(6)), [0], tb.RopeConfig(4, 1e4))
    with pytest.raises(Malformed, match="2 positions for 1 rows"):
        cb.rope(tb.Tensor.from_slice([4, 1], np.zeros(4)), [0, 1], tb.RopeConfig(4, 1e4))
    with pytest.raises(Malformed, match="id 9 is outside a table of 2 rows"):
        cb.get_rows(a, [0, 9])
    with pytest.raises(Malformed):
        cb.get_rows(a, [])  # Shape::new refuses the zero dimension
    with pytest.raises(Malformed):
        tb.Tensor.from_slice([2, 2], [1.0, 2.0, 3.0])
    with pytest.raises(Malformed):
        tb.Shape([1, 2, 3, 4, 5])
    with pytest.raises(Malformed):
        tb.Shape([3, 0])
