"""GPU parity: each CUDA kernel against the CPU oracle, through the C ABI.

Integer work, quantized bytes and indices must be bit-exact; so must every f32
result whose operation order the kernels reproduce (the quantized dot's tail,
norms, sequential dots). The only non-exact comparisons are the ones that go
through exp(), where the device rounds a double-precision exponential once and
the oracle calls the host libm; those are held to tolerance::F32_ULP-scaled
bounds stated at the assertion.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REDUCTION = 1e-5  # crates/llamd-core/src/tolerance.rs:39


@pytest.fixture(scope="module")
def be():
    from llamd_rs_b200 import backend

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    backend.stream_init()
    return backend


@pytest.fixture(scope="module")
def synth():
    from llamd_rs_b200 import synth

    return synth


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bit_equal(got, want, what=""):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    bad = np.flatnonzero(bits(got).ravel() != bits(want).ravel())
    assert bad.size == 0, f"{what}: {bad.size} of {got.size} differ, first at {bad[0]}: gpu {got.ravel()[bad[0]]!r} cpu {want.ravel()[bad[0]]!r}"


# ---- device discovery -------------------------------------------------------
def test_device_info(be):
    info = be.device_info(0)
    assert info.sm_count > 0 and info.warp_size == 32 and info.total_mem > 0
    assert info.arch.startswith("sm_")
    with pytest.raises(be.Malformed):
        be.device_info(be.device_count())


# ---- weights: the repack is a bit permutation -------------------------------
@pytest.mark.parametrize("rows,blocks", [(1, 1), (7, 3), (7, 5), (33, 8), (64, 16)])
def test_repack_round_trip_and_dequantize(be, orc, synth, rows, blocks):
    w = synth.q6k_blocks(rows * blocks, 11, "repack", rows, blocks)
    dw = be.DeviceWeights.upload(w, rows, blocks)
    assert np.array_equal(dw.unpack(), w), "tiled -> reference bytes must reproduce the upload"
    want = orc.dequantize(orc.Q6K, w, rows * blocks * 256)
    assert_bit_equal(dw.dequantize(), want, "dequantized weights")
    if rows * blocks > 2:
        assert_bit_equal(dw.dequantize(1, 2), want[256:768], "dequantize slice")


def test_dequantize_reference_kats(be, orc):
    """crates/llamd-quant/src/lib.rs:277-307 through the device layout."""
    blk = np.zeros(210, np.uint8)
    blk[192] = 1
    blk[208:210] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    assert be.DeviceWeights.upload(blk, 1, 1).dequantize()[0] == -32.0
    blk[0] = 0x05
    blk[128] = 0b11
    assert be.DeviceWeights.upload(blk, 1, 1).dequantize()[0] == 21.0


def test_upload_refuses_short_weights(be):
    with pytest.raises(be.Malformed):
        be.DeviceWeights.upload(np.zeros(10, np.uint8), 1, 1)
    with pytest.raises(be.Malformed):
        be.matvec_q6k(np.zeros(0, np.uint8), [], [], 0)


def test_q8_0_repack_and_dequantize(be, orc, synth):
    rows, blocks = 37, 5
    w = synth.q8_0_blocks(rows * blocks, 5, "q80")
    dw = be.Q80Weights.upload(w, rows, blocks)
    want = orc.dequantize(orc.Q8_0, w, rows * blocks * 32).reshape(rows, blocks * 32)
    assert_bit_equal(dw.dequantize(), want, "q8_0 dequantize")


# ---- Q8_K quantizer: crates/llamd-testing/tests/grouped_expert.rs:226-260 ----
def test_device_quantization_is_identical_to_the_host(be, orc):
    i = np.arange(256, dtype=np.float32)
    x = np.concatenate([
        np.sin(i * np.float32(0.11)) * np.float32(3.0),            # mixed
        -np.abs(np.cos(i * np.float32(0.07))) * np.float32(2.0),   # negative peak
        np.zeros(256, np.float32),                                  # all zero
        np.where(np.arange(256) % 2 == 0, 0.5, -0.5).astype(np.float32),  # ties
        np.where(np.arange(256) == 0, -8.0, 8.0).astype(np.float32),      # clamp
    ]).astype(np.float32)
    hq, hd, hb = orc.quantize_q8k(x)
    gq, gd, gb = be.quantize_q8k_on_device(x)
    assert_bit_equal(gd, hd, "block scales")
    assert np.array_equal(gq, hq), f"{np.count_nonzero(gq != hq)} quants differ"
    assert np.array_equal(gb, hb), "bsums"


def test_quantizer_on_random_and_tied_peaks(be, orc, synth):
    x = synth.normal_f32(256 * 64, 3, "q8k")
    x[256 + 5] = 7.0
    x[256 + 200] = -7.0          # equal magnitude later in the block: the first one wins
    x[512:768] = np.float32(1.5)  # every element ties for the peak
    hq, hd, hb = orc.quantize_q8k(x)
    gq, gd, gb = be.quantize_q8k_on_device(x)
    assert_bit_equal(gd, hd)
    assert np.array_equal(gq, hq) and np.array_equal(gb, hb)
    with pytest.raises(be.Malformed):
        be.quantize_q8k_on_device(np.zeros(100, np.float32))


# ---- matvec: crates/llamd-testing/tests/rocm_oracle.rs:78-108, planar.rs:42-87 --
@pytest.mark.parametrize("rows,blocks", [(1, 1), (7, 1), (7, 3), (5, 8), (40, 8), (33, 16), (100, 3), (300, 2)])
def test_matvec_is_bit_exact(be, orc, synth, rows, blocks):
    w = synth.q6k_blocks(rows * blocks, 21, "mv", rows, blocks)
    x = synth.normal_f32(blocks * 256, 21, "x", rows, blocks)
    qs, d, _ = orc.quantize_q8k(x)
    want = orc.matvec_q6k_q8k(w, qs, d, blocks * 256, rows)
    dw = be.DeviceWeights.upload(w, rows, blocks)
    assert_bit_equal(dw.matvec(qs, d), want, f"matvec {rows}x{blocks}")
    assert_bit_equal(be.matvec_q6k(w, qs, d, rows), want, "upload-per-call form")
    assert_bit_equal(dw.matvec_f32(x)[0], want, "f32-in form (device quantizer)")


def test_matvec_config0(be, orc, synth):
    """2048 x 2048 Q6_K, x ~ N(0,1), seed 0."""
    rows, blocks = 2048, 8
    w = synth.q6k_blocks(rows * blocks, 0, "config0")
    x = synth.normal_f32(2048, 0, "config0.x")
    want = orc.matvec_q6k(w, x, 2048, rows, threads=8)
    dw = be.DeviceWeights.upload(w, rows, blocks)
    assert_bit_equal(dw.matvec_f32(x)[0], want, "config 0")
    # The reference's other CPU path (dequantize, then f32 dot) is a different
    # algorithm; it must agree to what Q8_K allows, measured against the size
    # of the summed terms as crates/llamd-quant/src/dot.rs:311-321 does.
    f32_path = orc.matvec_dequant(orc.Q6K, w, x, 2048, rows, threads=8)
    wf = np.abs(orc.dequantize(orc.Q6K, w, rows * 2048).reshape(rows, 2048))
    scale = np.maximum((wf * np.abs(x)[None, :]).sum(1), 1e-6)
    assert np.max(np.abs(f32_path - want) / scale) < 5e-3


@pytest.mark.parametrize("nseq", [2, 4, 8])
@pytest.mark.parametrize("rows,blocks", [(70, 8), (45, 3), (20, 16)])
def test_batched_matvec_equals_single(be, orc, synth, rows, blocks, nseq):
    w = synth.q6k_blocks(rows * blocks, 31, "mvb", rows, blocks)
    x = synth.normal_f32(nseq * blocks * 256, 31, "xb", nseq)
    dw = be.DeviceWeights.upload(w, rows, blocks)
    got = dw.matvec_f32(x, nseq)
    for s in range(nseq):
        want = orc.matvec_q6k(w, x[s * blocks * 256:(s + 1) * blocks * 256], blocks * 256, rows)
        assert_bit_equal(got[s], want, f"sequence {s} of {nseq}")


# ---- grouped: crates/llamd-testing/tests/grouped_expert.rs:66-224 -----------
def test_grouped_equals_ungrouped_bit_exactly(be, orc, synth):
    n_expert, rows, blocks = 6, 48, 8
    w = synth.q6k_blocks(n_expert * rows * blocks, 41, "grp")
    x = synth.normal_f32(blocks * 256, 41, "grp.x")
    qs, d, _ = orc.quantize_q8k(x)
    dw = be.DeviceWeights.upload(w, n_expert * rows, blocks)
    ids = [4, 0, 5, 2]
    got = dw.matvec_grouped(qs, d, ids, rows)
    per = rows * blocks * 210
    for slot, e in enumerate(ids):
        want = orc.matvec_q6k_q8k(w[e * per:(e + 1) * per], qs, d, blocks * 256, rows)
        assert_bit_equal(got[slot], want, f"slot {slot} expert {e}")
        single = be.DeviceWeights.upload(w[e * per:(e + 1) * per], rows, blocks)
        assert_bit_equal(got[slot], single.matvec(qs, d), "grouped == ungrouped on the device")


def test_grouped_repeated_expert_and_bad_ids(be, orc, synth):
    n_expert, rows, blocks = 4, 16, 3
    w = synth.q6k_blocks(n_expert * rows * blocks, 42, "grp2")
    x = synth.normal_f32(blocks * 256, 42, "grp2.x")
    qs, d, _ = orc.quantize_q8k(x)
    dw = be.DeviceWeights.upload(w, n_expert * rows, blocks)
    got = dw.matvec_grouped(qs, d, [1, 1, 3], rows)
    assert_bit_equal(got[0], got[1], "the same expert twice gives the same rows")
    for bad in ([-1], [n_expert], [0, 99]):
        with pytest.raises(be.Malformed):
            dw.matvec_grouped(qs, d, bad, rows)
    with pytest.raises(be.Malformed):
        dw.matvec_grouped(qs, d, [0], rows + 1)  # non-divisor
    with pytest.raises(be.Malformed):
        dw.matvec_grouped(qs, d, [], rows)
    with pytest.raises(be.ShapeError):
        dw.matvec(qs[:256], d[:1])


# ---- Q8_0 matvec (no device kernel in the reference; CPU path model.rs:253-263) --
@pytest.mark.parametrize("rows,k,nseq", [
    (77, 512, 1), (77, 512, 3),   # two 8-block chunks, a ragged last row tile
    (33, 96, 2),                  # three blocks: less than one chunk
    (256, 2080, 1),               # 65 blocks: eight chunks and one block more
    (64, 1024, 8),                # one chain warp per sequence
    (40, 14336, 3),               # activations too large to sit beside the staged weights: the thread-per-row form
])
def test_q8_0_matvec_is_bit_exact(be, orc, synth, rows, k, nseq):
    w = synth.q8_0_blocks(rows * k // 32, 51, "q80mv", rows, k)
    x = synth.normal_f32(nseq * k, 51, "q80.x", rows, k)
    dw = be.Q80Weights.upload(w, rows, k // 32)
    got = dw.matvec_f32(x, nseq)
    for s in range(nseq):
        want = orc.matvec_dequant(orc.Q8_0, w, x[s * k:(s + 1) * k], k, rows)
        assert_bit_equal(got[s], want, f"q8_0 {rows}x{k} sequence {s}")


# ---- many tokens at once: the prefill kernels --------------------------------
@pytest.mark.parametrize("ntok", [1, 7, 8, 9, 37])
def test_matvec_tokens_equals_per_token_matvec(be, orc, synth, ntok):
    from llamd_rs_b200 import ops

    k, rows = 512, (70, 24, 24)
    ws = [synth.q6k_blocks(r * k // 256, 61, "mt", i) for i, r in enumerate(rows)]
    dws = [be.DeviceWeights.upload(w, r, k // 256) for w, r in zip(ws, rows)]
    x = synth.normal_f32(ntok * k, 61, "mt.x", ntok).reshape(ntok, k)
    got = ops.matvec_tokens(dws, x)
    for w, r, g in zip(ws, rows, got):
        for t in range(ntok):
            assert_bit_equal(g[t], orc.matvec_q6k(w, x[t], k, r), f"token {t}")
    assert_bit_equal(ops.matvec_tokens(dws[:1], x)[0], got[0], "one matrix alone")
    for a, b in zip(ops.matvec_tokens(dws, x, gemm=True), got):
        assert_bit_equal(a, b, "tensor-path GEMM == dp4a matvec")


@pytest.mark.parametrize("ntok,n_used", [(1, 2), (5, 2), (40, 3), (64, 8)])
def test_expert_major_equals_token_major(be, orc, synth, ntok, n_used):
    """crates/llamd-testing/tests/vulkan_prefill.rs:268-330: the expert-major path gives exactly what the
    per-token grouped matvec gives."""
    from llamd_rs_b200 import ops

    n_expert, rows, k = 16, 48, 512
    per = rows * k // 256 * 210
    wa = synth.q6k_blocks(n_expert * rows * k // 256, 62, "em.a")
    wb = synth.q6k_blocks(n_expert * rows * k // 256, 62, "em.b")
    da, db = be.DeviceWeights.upload(wa, n_expert * rows, k // 256), be.DeviceWeights.upload(wb, n_expert * rows, k // 256)
    rng = np.random.default_rng(ntok)
    ids = np.stack([rng.permutation(n_expert)[:n_used] for _ in range(ntok)]).astype(np.int32)
    if ntok >= 40:
        ids[:, 0] = 3  # one hot expert: more than 8 pairs, so its work is cut into several items
    x = synth.normal_f32(ntok * k, 62, "em.x", ntok).reshape(ntok, k)
    ga, gb = ops.expert_major([da, db], x, ids, rows)
    for t in range(ntok):
        for s_ in range(n_used):
            e = int(ids[t, s_])
            assert_bit_equal(ga[t * n_used + s_], orc.matvec_q6k(wa[e * per:(e + 1) * per], x[t], k, rows), f"gate pair ({t},{s_})")
            assert_bit_equal(gb[t * n_used + s_], orc.matvec_q6k(wb[e * per:(e + 1) * per], x[t], k, rows), f"up pair ({t},{s_})")
    # down: every pair has its own activation
    xs = synth.normal_f32(ntok * n_used * k, 62, "em.xs", ntok).reshape(ntok * n_used, k)
    (gd,) = ops.expert_major([da], xs, ids, rows, by_slot=True)
    for p_ in range(ntok * n_used):
        e = int(ids.ravel()[p_])
        assert_bit_equal(gd[p_], orc.matvec_q6k(wa[e * per:(e + 1) * per], xs[p_], k, rows), f"down pair {p_}")
    # the integer tensor path gives the same bits
    ta, tb = ops.expert_major([da, db], x, ids, rows, gemm=True)
    assert_bit_equal(ta, ga, "expert GEMM gate")
    assert_bit_equal(tb, gb, "expert GEMM up")
    (td,) = ops.expert_major([da], xs, ids, rows, by_slot=True, gemm=True)
    assert_bit_equal(td, gd, "expert GEMM down")
    with pytest.raises(be.Malformed):
        ops.expert_major([da], x, np.full((ntok, n_used), n_expert, np.int32), rows)


# ---- matvecs with the activation's quantization (and SiLU) fused in -----------
@pytest.mark.parametrize("nseq", [1, 3, 8])
def test_matvec_f32act_equals_quantize_then_matvec(be, orc, synth, nseq):
    from llamd_rs_b200 import ops

    rows, k = 90, 1024
    w = synth.q6k_blocks(rows * k // 256, 71, "f32act")
    x = synth.normal_f32(nseq * k, 71, "f32act.x", nseq).reshape(nseq, k)
    x[0, 256:512] = 0.0  # an all-zero block: d = 0
    dw = be.DeviceWeights.upload(w, rows, k // 256)
    got = ops.matvec_f32act(dw, x)
    for s_ in range(nseq):
        assert_bit_equal(got[s_], orc.matvec_q6k(w, x[s_], k, rows), f"sequence {s_}")


def test_down_projection_with_fused_silu(be, orc, synth):
    from llamd_rs_b200 import ops

    n_expert, rows, k = 6, 64, 768
    per = rows * k // 256 * 210
    w = synth.q6k_blocks(n_expert * rows * k // 256, 72, "pasilu")
    dw = be.DeviceWeights.upload(w, n_expert * rows, k // 256)
    ids = [5, 0, 3, 3]
    gate = synth.normal_f32(len(ids) * k, 72, "g").reshape(len(ids), k) * np.float32(2.0)
    up = synth.normal_f32(len(ids) * k, 72, "u").reshape(len(ids), k)
    got = ops.matvec_grouped_pa_silu(dw, ids, gate, up, rows)
    act = ops.silu_mul(gate.ravel(), up.ravel()).reshape(len(ids), k)  # the device's own activation (exp differs from libm by <= 1 ulp)
    for s_, e in enumerate(ids):
        assert_bit_equal(got[s_], orc.matvec_q6k(w[e * per:(e + 1) * per], act[s_], k, rows), f"slot {s_}")


def test_gemm_rows_not_a_multiple_of_16_and_odd_blocks(be, orc, synth):
    from llamd_rs_b200 import ops

    for rows, k, ntok in ((37, 768, 11), (5, 256, 3), (100, 4096, 9)):
        w = synth.q6k_blocks(rows * k // 256, 81, "gemm", rows)
        dw = be.DeviceWeights.upload(w, rows, k // 256)
        x = synth.normal_f32(ntok * k, 81, "gemm.x", rows).reshape(ntok, k)
        (got,) = ops.matvec_tokens([dw], x, gemm=True)
        for t in range(ntok):
            assert_bit_equal(got[t], orc.matvec_q6k(w, x[t], k, rows), f"{rows}x{k} token {t}")
