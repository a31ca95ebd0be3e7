"""The oracle against the reference's own known-answer tests.

Each test restates one unit test of the reference (file:line in its docstring)
so that the C restatement in ``oracle/llamd_oracle.c`` is pinned by the same
vectors that pin the reference.
"""
import math

import numpy as np
import pytest

QK_K = 256
Q6K = 210


def f16(orc, v):
    return np.frombuffer(np.uint16(orc.f32_to_f16(v)).tobytes(), dtype=np.uint8)


def close(a, b, tol):
    """llamd_core::tolerance::close (crates/llamd-core/src/tolerance.rs:116-129)."""
    a, b = np.float32(a), np.float32(b)
    if tol == 0.0:
        return a.tobytes() == b.tobytes()
    if math.isnan(a) or math.isnan(b):
        return math.isnan(a) and math.isnan(b)
    return abs(a - b) / max(abs(a), abs(b), 1.0) <= tol


F32_ULP, REDUCTION, ATTENTION = 1.2e-7, 1e-5, 1e-5


# ---- crates/llamd-quant/src/lib.rs:235-323
def test_block_sizes_and_type_ids(orc):
    assert orc.bytes_for(orc.Q6K, 256) == 210
    assert orc.bytes_for(orc.Q8_0, 32) == 34
    assert orc.bytes_for(orc.Q6K, 512) == 420
    assert orc.bytes_for(orc.Q6K, 100) == -2  # partial_blocks_are_refused
    assert orc.bytes_for(12, 256) == -1  # an unimplemented ggml type says so
    assert (orc.F32, orc.F16, orc.Q8_0, orc.Q6K) == (0, 1, 8, 14)


def test_f16_round_trip_every_bit_pattern(orc):
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([orc.f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    assert got.tobytes() == want.tobytes() or np.array_equal(
        got[~np.isnan(want)].view(np.uint32), want[~np.isnan(want)].view(np.uint32))
    for v in (2.0, 1.0, 0.5, 1e-3, 6.1e-5, 3e-8, -0.0156, 65504.0):
        assert orc.f32_to_f16(v) == int(np.float16(np.float32(v)).view(np.uint16))


def test_q8_0_dequantizes_by_hand(orc):
    blk = np.zeros(34, np.uint8)
    blk[0:2] = f16(orc, 2.0)
    blk[2] = 1
    blk[3] = 0xFF
    out = orc.dequantize(orc.Q8_0, blk, 32)
    assert out[0] == 2.0 and out[1] == -2.0 and np.all(out[2:] == 0.0)


def test_q6k_centres_on_minus_32(orc):
    blk = np.zeros(Q6K, np.uint8)
    blk[192] = 1
    blk[208:210] = f16(orc, 1.0)
    out = orc.dequantize(orc.Q6K, blk, 256)
    assert out.size == 256 and out[0] == -32.0


def test_q6k_reads_high_bits_from_qh(orc):
    blk = np.zeros(Q6K, np.uint8)
    blk[0] = 0x05
    blk[128] = 0b11
    blk[192] = 1
    blk[208:210] = f16(orc, 1.0)
    assert orc.dequantize(orc.Q6K, blk, 256)[0] == 21.0


def test_short_input_is_refused(orc):
    with pytest.raises(ValueError):
        orc.dequantize(orc.Q6K, np.zeros(10, np.uint8), 256)


# ---- crates/llamd-quant/src/dot.rs:204-346
def test_rounding_is_half_to_even(orc):
    for v, w in [(0.5, 0), (1.5, 2), (2.5, 2), (-0.5, 0), (-1.5, -2), (-2.5, -2)]:
        assert orc.nearest_int(v) == w


def test_peak_magnitude_maps_to_minus_127(orc):
    for peak in (5.0, -5.0):
        v = np.full(256, 0.1, np.float32)
        v[7] = peak
        assert orc.quantize_q8k(v)[0][7] == -127


def test_all_zero_block_has_no_scale(orc):
    qs, d, bs = orc.quantize_q8k(np.zeros(256, np.float32))
    assert d[0] == 0.0 and np.all(qs == 0) and np.all(bs == 0)


def test_bsums_are_group_sums(orc):
    v = np.sin(np.arange(256, dtype=np.float32) * np.float32(0.01)).astype(np.float32)
    qs, d, bs = orc.quantize_q8k(v)
    assert np.array_equal(bs, qs.astype(np.int16).reshape(16, 16).sum(1))


def q6k_block(orc, codes, scale, d):
    """dot.rs:258-282"""
    blk = np.zeros(Q6K, np.uint8)
    for half in range(2):
        ql, qh, o = half * 64, 128 + half * 32, half * 128
        for l in range(32):
            c0, c1, c2, c3 = (int(codes[o + l]), int(codes[o + l + 32]), int(codes[o + l + 64]), int(codes[o + l + 96]))
            blk[ql + l] = (c0 & 0xF) | ((c2 & 0xF) << 4)
            blk[ql + l + 32] = (c1 & 0xF) | ((c3 & 0xF) << 4)
            blk[qh + l] = (c0 >> 4) | ((c1 >> 4) << 2) | ((c2 >> 4) << 4) | ((c3 >> 4) << 6)
    blk[192:208] = np.uint8(scale & 0xFF)
    blk[208:210] = f16(orc, d)
    return blk


def test_dot_agrees_with_dequantize_then_multiply(orc):
    codes = np.array([32 + (i % 7) - 3 for i in range(256)], np.uint8)
    w = q6k_block(orc, codes, 2, 0.5)
    x = np.sin(np.arange(256, dtype=np.float32) * np.float32(0.05)).astype(np.float32)
    qs, d, _ = orc.quantize_q8k(x)
    quantized = orc.dot_q6k_q8k(w, qs, d, 256)
    wf = orc.dequantize(orc.Q6K, w, 256)
    exact = float(np.sum(wf * x, dtype=np.float32))
    scale = max(float(np.sum(np.abs(wf * x))), 1e-6)
    assert abs(quantized - exact) / scale < 5e-3


def test_zero_weight_block_gives_zero(orc):
    w = q6k_block(orc, np.full(256, 32, np.uint8), 1, 1.0)
    qs, d, _ = orc.quantize_q8k(np.arange(256, dtype=np.float32))
    assert orc.dot_q6k_q8k(w, qs, d, 256) == 0.0


def test_multiple_blocks_accumulate(orc):
    w1 = q6k_block(orc, np.full(256, 33, np.uint8), 1, 1.0)
    w = np.concatenate([w1, w1])
    qs, d, _ = orc.quantize_q8k(np.ones(512, np.float32))
    one = orc.dot_q6k_q8k(w1, qs[:256], d[:1], 256)
    two = orc.dot_q6k_q8k(w, qs, d, 512)
    assert abs(two - 2.0 * one) < 1e-3 * max(abs(one), 1.0)


def test_dot_matches_a_pure_python_restatement(orc):
    """Independent check of the integer core and the 8-lane f32 tail."""
    rng = np.random.default_rng(3)
    nb = 3
    w = rng.integers(0, 256, nb * Q6K, dtype=np.uint8)
    for b in range(nb):
        w[b * Q6K + 208: b * Q6K + 210] = f16(orc, 0.0123 * (b + 1))
    x = rng.standard_normal(nb * 256).astype(np.float32)
    qs, d, _ = orc.quantize_q8k(x)
    sums = [np.float32(0)] * 8
    for b in range(nb):
        blk = w[b * Q6K:(b + 1) * Q6K]
        aux8 = np.zeros(256, np.int32)
        for half in range(2):
            for l in range(32):
                h, lo0, lo1 = int(blk[128 + half * 32 + l]), int(blk[half * 64 + l]), int(blk[half * 64 + l + 32])
                o = half * 128
                aux8[o + l] = ((lo0 & 15) | ((h & 3) << 4)) - 32
                aux8[o + l + 32] = ((lo1 & 15) | (((h >> 2) & 3) << 4)) - 32
                aux8[o + l + 64] = ((lo0 >> 4) | (((h >> 4) & 3) << 4)) - 32
                aux8[o + l + 96] = ((lo1 >> 4) | (((h >> 6) & 3) << 4)) - 32
        aux32 = [0] * 8
        for j in range(16):
            sc = int(np.int8(blk[192 + j]))
            for e in range(16):
                aux32[e % 8] += sc * int(qs[b * 256 + j * 16 + e]) * int(aux8[j * 16 + e])
        dd = np.float32(orc.f16_to_f32(int(blk[208]) | (int(blk[209]) << 8))) * d[b]
        for l in range(8):
            sums[l] = np.float32(sums[l] + np.float32(dd * np.float32(aux32[l])))
    total = np.float32(0)
    for l in range(8):
        total = np.float32(total + sums[l])
    assert close(orc.dot_q6k_q8k(w, qs, d, nb * 256), total, 0.0)


# ---- crates/llamd-quant/src/dot.rs:426-483
def test_planar_repack_is_a_permutation(orc):
    rows, blocks = 7, 5
    src = (np.arange(rows * blocks * Q6K) % 251).astype(np.uint8)
    out, off = orc.repack_q6k_planar(src, rows, blocks)
    assert out.size == src.size == off[4]
    assert np.array_equal(np.bincount(src, minlength=256), np.bincount(out, minlength=256))
    i = 3
    blk = src[i * Q6K:(i + 1) * Q6K]
    assert np.array_equal(out[off[0] + i * 128: off[0] + i * 128 + 128], blk[:128])
    assert np.array_equal(out[off[1] + i * 64: off[1] + i * 64 + 64], blk[128:192])
    assert np.array_equal(out[off[2] + i * 16: off[2] + i * 16 + 16], blk[192:208])
    assert np.array_equal(out[off[3] + i * 2: off[3] + i * 2 + 2], blk[208:210])
    with pytest.raises(ValueError):
        orc.repack_q6k_planar(np.zeros(10, np.uint8), 1, 1)


# ---- crates/llamd-models/src/moe.rs:120-246
def test_route_selects_best_first(orc):
    assert list(orc.route([0.1, 5.0, 0.2, 3.0, 0.3], 2)["experts"]) == [1, 3]


def test_route_weights_sum_to_one(orc):
    r = orc.route([1, 2, 3, 4, 5, 6, 7, 8], 3)
    assert close(np.sum(r["weights"], dtype=np.float32), 1.0, ATTENTION)
    assert r["weights"][0] > r["weights"][1] > r["weights"][2]


def test_route_renormalises_not_resoftmaxes(orc):
    r = orc.route([10.0, 9.0, 0.0, 0.0], 2)
    assert close(r["weights"][0], 0.7310586, ATTENTION)
    assert close(r["weights"][1], 0.2689414, ATTENTION)


def test_route_ties_break_low(orc):
    for _ in range(8):
        assert list(orc.route([1.0, 1.0, 1.0, 1.0], 2)["experts"]) == [0, 1]


def test_route_real_shape(orc):
    logits = (np.sin(np.arange(128, dtype=np.float32) * np.float32(0.37)) * np.float32(3.0)).astype(np.float32)
    r = orc.route(logits, 8)
    assert len(set(r["experts"].tolist())) == 8
    assert close(np.sum(r["weights"], dtype=np.float32), 1.0, ATTENTION)
    # same choice as a plain argsort on the logits (softmax is monotonic here)
    assert set(r["experts"].tolist()) == set(np.argsort(-logits, kind="stable")[:8].tolist())


def test_route_degenerate_and_impossible(orc):
    r = orc.route([0.0, -800.0, -800.0, -800.0], 3)
    assert np.all(np.isfinite(r["weights"]))
    for bad in (0, 3):
        with pytest.raises(ValueError):
            orc.route([1.0, 2.0], bad)


# ---- crates/llamd-cpu/src/lib.rs:236-368
def test_rms_norm(orc):
    out = orc.rms_norm(np.array([3.0, 4.0], np.float32), 0.0)
    rms = np.sqrt(np.float32(12.5))
    assert close(out[0], 3.0 / rms, F32_ULP) and close(out[1], 4.0 / rms, F32_ULP)
    out = orc.rms_norm(np.array([[3.0, 4.0], [300.0, 400.0]], np.float32), 0.0)
    assert close(out[0, 0], out[1, 0], ATTENTION) and close(out[0, 1], out[1, 1], ATTENTION)


def test_softmax(orc):
    out = orc.softmax(np.array([1.0, 2.0, 3.0], np.float32))
    assert close(out.sum(dtype=np.float32), 1.0, F32_ULP)
    big = orc.softmax(np.array([1000.0, 1001.0, 1002.0], np.float32))
    assert np.all(np.isfinite(big))
    assert all(close(a, c, ATTENTION) for a, c in zip(out, big))


def test_silu(orc):
    out = orc.silu(np.array([0.0, 1.0, -1.0], np.float32))
    assert close(out[0], 0.0, F32_ULP)
    assert close(out[1], 1.0 / (1.0 + math.exp(-1.0)), F32_ULP)
    assert -1.0 < out[2] < 0.0


def test_matmul_is_a_row_dot(orc):
    w = np.array([[1, 2], [3, 4], [5, 6]], np.float32)
    out = orc.matmul(w, np.array([[1, 1]], np.float32))
    assert out.shape == (1, 3) and out.tolist() == [[3.0, 7.0, 11.0]]


def test_rope(orc):
    x = np.array([1, 2, 3, 4], np.float32)
    out = orc.rope(x[None], [0], 4, 10000.0)[0]
    assert all(close(a, c, F32_ULP) for a, c in zip(x, out))
    out = orc.rope(np.array([[1, 0, 0, 0]], np.float32), [1], 4, 10000.0)[0]
    assert close(out[0], math.cos(1.0), ATTENTION) and close(out[2], math.sin(1.0), ATTENTION)
    assert close(out[1], 0.0, ATTENTION)
    x = np.array([0.3, -1.2, 0.7, 2.0, -0.5, 1.1, 0.9, -0.2], np.float32)
    out = orc.rope(x[None], [37], 8, 1e7)[0]
    for i in range(4):
        assert close(math.hypot(x[i], x[i + 4]), math.hypot(out[i], out[i + 4]), ATTENTION)
    with pytest.raises(ValueError):
        orc.rope(np.zeros((1, 6), np.float32), [0], 3, 1e4)


def test_get_rows(orc):
    table = np.array([[1, 2], [3, 4], [5, 6]], np.float32)
    assert orc.get_rows(table, [2, 0]).tolist() == [[5, 6], [1, 2]]
    with pytest.raises(ValueError):
        orc.get_rows(table, [9])


# ---- crates/llamd-runtime/src/attention.rs:140-247
def test_attend_single_position_returns_value(orc):
    out = orc.attend([0.5] * 4, [0.25] * 4, [7, 8, 9, 10], 1, 1, 1, 4)
    assert all(close(o, e, ATTENTION) for o, e in zip(out, [7, 8, 9, 10]))


def test_attend_gqa_integer_division(orc):
    out = orc.attend([1, 0] * 4, [1, 0, 1, 0], [100, 100, 200, 200], 1, 4, 2, 2)
    assert [close(out[i], w, ATTENTION) for i, w in ((0, 100), (2, 100), (4, 200), (6, 200))] == [True] * 4


def test_attend_scale(orc):
    out = orc.attend([2, 0, 0, 0], [2, 0, 0, 0, 0, 2, 0, 0], [1, 0, 0, 0, 0, 0, 0, 0], 2, 1, 1, 4)
    want = math.exp(2.0) / (math.exp(2.0) + 1.0)
    assert close(out[0], want, ATTENTION)


def test_attend_large_logits_and_refusals(orc):
    out = orc.attend([100.0] * 4, [100.0] * 4 + [-100.0] * 4, [1.0] * 4 + [2.0] * 4, 2, 1, 1, 4)
    assert np.all(np.isfinite(out)) and close(out[0], 1.0, ATTENTION)
    with pytest.raises(ValueError):
        orc.attend([0.0] * 4, [0.0] * 4, [0.0] * 4, 1, 3, 2, 2)
    with pytest.raises(ValueError):
        orc.attend([0.0] * 3, [0.0] * 4, [0.0] * 4, 1, 1, 1, 4)
    with pytest.raises(ValueError):
        orc.attend([0.0] * 4, [0.0] * 4, [0.0] * 4, 0, 1, 1, 4)


def test_attend_real_shape(orc):
    n_head, n_head_kv, hd, n_kv = 32, 4, 128, 7
    q = np.sin(np.arange(n_head * hd, dtype=np.float32) * np.float32(0.01))
    k = np.cos(np.arange(n_kv * n_head_kv * hd, dtype=np.float32) * np.float32(0.02))
    v = np.sin(np.arange(n_kv * n_head_kv * hd, dtype=np.float32) * np.float32(0.03))
    out = orc.attend(q, k, v, n_kv, n_head, n_head_kv, hd)
    assert out.size == n_head * hd and np.all(np.isfinite(out))


# ---- matvec wrappers (crates/llamd-models/src/model.rs:241-318)
def test_matvec_q6k_is_quantize_then_row_dots(orc):
    rng = np.random.default_rng(1)
    rows, nb = 7, 3
    w = rng.integers(0, 256, rows * nb * Q6K, dtype=np.uint8)
    for i in range(rows * nb):
        w[i * Q6K + 208: i * Q6K + 210] = f16(orc, 0.01)
    x = rng.standard_normal(nb * 256).astype(np.float32)
    qs, d, _ = orc.quantize_q8k(x)
    want = [orc.dot_q6k_q8k(w[r * nb * Q6K:(r + 1) * nb * Q6K], qs, d, nb * 256) for r in range(rows)]
    for th in (1, 3):
        got = orc.matvec_q6k(w, x, nb * 256, rows, threads=th)
        assert got.tolist() == want


def test_matvec_dequant_q8_0_is_sequential_f32(orc):
    rng = np.random.default_rng(2)
    rows, k = 5, 64
    w = rng.integers(0, 256, rows * (k // 32) * 34, dtype=np.uint8)
    for i in range(rows * k // 32):
        w[i * 34: i * 34 + 2] = f16(orc, 0.02)
    x = rng.standard_normal(k).astype(np.float32)
    wf = orc.dequantize(orc.Q8_0, w, rows * k).reshape(rows, k)
    got = orc.matvec_dequant(orc.Q8_0, w, x, k, rows)
    for r in range(rows):
        acc = np.float32(-0.0)
        for t in range(k):
            acc = np.float32(acc + np.float32(wf[r, t] * x[t]))
        assert close(got[r], acc, 0.0)


def test_round_to_f16_is_ieee_nearest_even():
    """The oracle's f16-store mode of the KV cache rounds as numpy's float16 conversion does (IEEE binary16, ties to
    even, overflow to infinity, subnormals kept), including the midpoints."""
    import oracle

    L = oracle.lib()
    rng = np.random.default_rng(5)
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-6, 1e-4, 1e-2, 1.0, 100.0, 3e4)]
                        + [np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 65536.0, -65520.0, 6.1e-5, 6.103515625e-5, 5.96e-8, 2.98e-8,
                                     2.9802322e-8, 8.9e-8, 1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11, np.inf, -np.inf], np.float32)])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).astype(np.float32)
    got = np.array([L.orc_round_to_f16(float(v)) for v in xs], np.float32)
    assert np.array_equal(want.view(np.uint32), got.view(np.uint32))
