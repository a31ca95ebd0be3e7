"""GPU parity of the f32 ops around the matvecs (router, norms, RoPE,
attention, SiLU, combine, argmax, scatter plan) against the oracle.

Everything without an exponential is bit-exact. Where exp() is involved the
device rounds a double-precision exponential once while the oracle calls the
host libm; the two differ by one ulp on a small fraction of inputs, so those
outputs are compared at tolerance::ATTENTION (1e-5, crates/llamd-core/src/tolerance.rs:97)
and the discrete results (expert ids) must still match on these inputs.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ATTENTION = 1e-5
F32_ULP = 1.2e-7


@pytest.fixture(scope="module")
def ops():
    from llamd_rs_b200 import backend, ops

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    backend.stream_init()
    return ops


@pytest.fixture(scope="module")
def synth():
    from llamd_rs_b200 import synth

    return synth


def bit_equal(a, b):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def max_dev(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.maximum(np.abs(a), np.abs(b)), 1.0)))


def test_rms_norm_is_bit_exact(ops, orc, synth):
    x = synth.normal_f32(3 * 2048, 1, "rms").reshape(3, 2048)
    w = synth.normal_f32(2048, 1, "rms.w")
    want = orc.mul(orc.rms_norm(x, 1e-6), np.tile(w, 3)).reshape(3, 2048)
    assert bit_equal(ops.rms_norm_mul(x, w, 1e-6), want)
    out, qs, d = ops.rms_norm_quant(x, w, 1e-6)
    assert bit_equal(out, want)
    hq, hd, _ = orc.quantize_q8k(want)
    assert np.array_equal(qs, hq) and bit_equal(d, hd)
    r = synth.normal_f32(3 * 2048, 1, "rms.r").reshape(3, 2048)
    out, qs, d, s = ops.rms_norm_quant(x, w, 1e-6, residual=r)
    assert bit_equal(s, orc.add(x, r).reshape(3, 2048))
    assert bit_equal(out, orc.mul(orc.rms_norm(s, 1e-6), np.tile(w, 3)).reshape(3, 2048))
    # crates/llamd-cpu/src/lib.rs:237-244
    got = ops.rms_norm_mul(np.array([3.0, 4.0, 0.0, 0.0], np.float32), np.ones(4, np.float32), 0.0)
    assert bit_equal(got, orc.rms_norm(np.array([3.0, 4.0, 0.0, 0.0], np.float32), 0.0))


def test_head_norm_and_rope_are_bit_exact(ops, orc, synth):
    n_head, hd = 8, 128
    x = synth.normal_f32(n_head * hd, 2, "rope")
    w = synth.normal_f32(hd, 2, "rope.w")
    normed = orc.rms_norm(x.reshape(n_head, hd), 1e-6) * 0 + orc.mul(orc.rms_norm(x.reshape(n_head, hd), 1e-6).ravel(), np.tile(w, n_head)).reshape(n_head, hd)
    assert bit_equal(ops.head_rms_norm_mul(x, w, n_head, hd, 1e-6), normed.ravel())
    for pos in (0, 1, 37, 700):
        want = orc.rope(normed.reshape(1, -1), [pos], hd, 1e7)[0]
        assert bit_equal(ops.norm_rope(x, w, n_head, hd, pos, 1e7, 1e-6), want), f"pos {pos}"
        assert bit_equal(ops.norm_rope(x, None, n_head, hd, pos, 1e7, 1e-6), orc.rope(x.reshape(1, -1), [pos], hd, 1e7)[0])
    # crates/llamd-cpu/src/lib.rs:314-322: position 0 is the identity
    assert bit_equal(ops.norm_rope(x, None, n_head, hd, 0, 1e4, 0.0), x)
    tab = ops.rope_table(5, 8, 1e7)
    s, c = orc.rope_angles(3, 8, 1e7)
    assert bit_equal(tab[3, :, 0], s) and bit_equal(tab[3, :, 1], c)


@pytest.mark.parametrize("n_kv", [1, 7, 64, 65, 200, 513])
def test_attention_matches(ops, orc, synth, n_kv):
    n_head, n_head_kv, hd = 32, 4, 128
    q = synth.normal_f32(n_head * hd, 3, "att.q", n_kv)
    k = synth.normal_f32(n_kv * n_head_kv * hd, 3, "att.k", n_kv)
    v = synth.normal_f32(n_kv * n_head_kv * hd, 3, "att.v", n_kv)
    want = orc.attend(q, k, v, n_kv, n_head, n_head_kv, hd)
    got = ops.attention(q, k, v, n_kv, n_head, n_head_kv, hd)
    if n_kv == 1:
        assert bit_equal(got, want), "a single key gives exactly its value"
    assert max_dev(got, want) <= ATTENTION
    split = ops.attention(q, k, v, n_kv, n_head, n_head_kv, hd, scores=True)
    assert bit_equal(split, got), "the split-over-CTAs variant keeps every sum in order"


@pytest.mark.parametrize("n_head,n_head_kv,hd,base,ntok,max_kv", [
    (8, 2, 128, 0, 70, 128),      # ragged token and position tiles, first tile of a prompt
    (4, 2, 64, 37, 33, 96),       # a later tile: 37 positions of context before it
    (4, 1, 128, 100, 1, 104),     # a single token with context
    (4, 4, 64, 0, 96, 100),       # no grouping
    (4, 2, 96, 0, 9, 16),         # a head_dim the tiled kernels do not cover: falls through
    (4, 2, 64, 0, 9, 18),         # max_kv not a multiple of 4: falls through
])
def test_attention_prefill_tile(ops, orc, synth, n_head, n_head_kv, hd, base, ntok, max_kv):
    """The register-tiled prefill attention equals the per-token kernels bit for bit and `attend` per token."""
    n_rows = base + ntok
    kv_dim = n_head_kv * hd
    q = synth.normal_f32(ntok * n_head * hd, 5, "attp.q", hd, ntok).reshape(ntok, -1)
    k = synth.normal_f32(n_rows * kv_dim, 5, "attp.k", hd, ntok)
    v = synth.normal_f32(n_rows * kv_dim, 5, "attp.v", hd, ntok)
    pos = np.arange(base, base + ntok, dtype=np.int32)
    got = ops.attention_prefill(q, k, v, pos, n_head, n_head_kv, hd, max_kv)
    per_token = ops.attention_prefill(q, k, v, pos, n_head, n_head_kv, hd, max_kv, tiled=False)
    assert bit_equal(got, per_token)
    for i in (0, ntok // 2, ntok - 1):
        n_kv = int(pos[i]) + 1
        want = orc.attend(q[i], k[: n_kv * kv_dim], v[: n_kv * kv_dim], n_kv, n_head, n_head_kv, hd)
        assert max_dev(got[i], want) <= ATTENTION
    # positions need not be consecutive or increasing
    perm = np.random.default_rng(1).permutation(ntok)
    got2 = ops.attention_prefill(q[perm], k, v, pos[perm], n_head, n_head_kv, hd, max_kv)
    assert bit_equal(got2, got[perm])


def test_attention_reference_kats(ops, orc):
    """crates/llamd-runtime/src/attention.rs:140-213"""
    out = ops.attention([0.5] * 4, [0.25] * 4, [7, 8, 9, 10], 1, 1, 1, 4)
    assert out.tolist() == [7.0, 8.0, 9.0, 10.0]
    out = ops.attention([1, 0, 0, 0] * 4, [1, 0, 0, 0, 1, 0, 0, 0], [100] * 4 + [200] * 4, 1, 4, 2, 4)
    assert out[0] == 100 and out[4] == 100 and out[8] == 200 and out[12] == 200, "GQA maps by integer division"
    out = ops.attention([2, 0, 0, 0], [2, 0, 0, 0, 0, 2, 0, 0], [1, 0, 0, 0, 0, 0, 0, 0], 2, 1, 1, 4)
    assert abs(out[0] - np.exp(2.0) / (np.exp(2.0) + 1.0)) < ATTENTION
    out = ops.attention([100.0] * 4, [100.0] * 4 + [-100.0] * 4, [1.0] * 4 + [2.0] * 4, 2, 1, 1, 4)
    assert np.all(np.isfinite(out)) and abs(out[0] - 1.0) < ATTENTION
    from llamd_rs_b200 import backend

    with pytest.raises(backend.Malformed):
        ops.attention([0.0] * 4, [0.0] * 4, [0.0] * 4, 1, 3, 2, 2)  # 3 does not group into 2
    with pytest.raises(backend.ShapeError):
        ops.attention([0.0] * 3, [0.0] * 4, [0.0] * 4, 1, 1, 1, 4)
    with pytest.raises(backend.Malformed):
        ops.attention([0.0] * 4, [], [], 0, 1, 1, 4)
    with pytest.raises(backend.Malformed):
        ops.attention([0.0] * 6, [0.0] * 4, [0.0] * 4, 1, 3, 2, 2)


def test_router_matches_route(ops, orc, synth):
    logits = synth.normal_f32(5 * 128, 4, "router").reshape(5, 128) * np.float32(2.0)
    ids, w, probs = ops.router(logits, 8)
    for s in range(5):
        r = orc.route(logits[s], 8)
        assert ids[s].tolist() == r["experts"].tolist(), f"sequence {s}"
        assert max_dev(w[s], r["weights"]) <= ATTENTION and max_dev(probs[s], r["probs"]) <= ATTENTION


def test_router_reference_kats(ops, orc):
    """crates/llamd-models/src/moe.rs:120-246"""
    from llamd_rs_b200 import backend

    assert ops.router([0.1, 5.0, 0.2, 3.0, 0.3], 2)[0][0].tolist() == [1, 3]
    ids, w, _ = ops.router([10.0, 9.0, 0.0, 0.0], 2)
    assert abs(w[0][0] - 0.7310586) < ATTENTION and abs(w[0][1] - 0.2689414) < ATTENTION
    for _ in range(4):
        assert ops.router([1.0, 1.0, 1.0, 1.0], 2)[0][0].tolist() == [0, 1], "ties break toward the lower index"
    ids, w, _ = ops.router([0.0, -800.0, -800.0, -800.0], 3)
    assert np.all(np.isfinite(w)) and ids[0][0] == 0
    assert ids[0].tolist() == [0, 1, 2], "equal (zero) probabilities are taken in index order"
    logits = (np.sin(np.arange(128, dtype=np.float32) * np.float32(0.37)) * np.float32(3.0)).astype(np.float32)
    ids, w, _ = ops.router(logits, 8)
    assert ids[0].tolist() == orc.route(logits, 8)["experts"].tolist() and len(set(ids[0].tolist())) == 8
    for bad in (0, 3):
        with pytest.raises(backend.Malformed):
            ops.router([1.0, 2.0], bad)


def test_router_matvec_logits_are_bit_exact(ops, orc, synth):
    ne, k = 128, 2048
    w = synth.normal_f32(ne * k, 5, "rw", std=0.02).reshape(ne, k)
    x = synth.normal_f32(3 * k, 5, "rx").reshape(3, k)
    logits, ids, wts = ops.router_matvec(w, x, 8)
    for s in range(3):
        want = orc.matvec_dequant(orc.F32, w, x[s], k, ne)
        assert bit_equal(logits[s], want), "router logits: sequential f32 dot"
        r = orc.route(want, 8)
        assert ids[s].tolist() == r["experts"].tolist()
        assert max_dev(wts[s], r["weights"]) <= ATTENTION
    assert bit_equal(ops.matvec_f32(w, x), np.stack([orc.matvec_dequant(orc.F32, w, x[s], k, ne) for s in range(3)]))


@pytest.mark.parametrize("rows,k,ntok", [(128, 2048, 37), (8, 256, 1), (50, 100, 19), (33, 68, 16)])
def test_matmul_f32_tokens(ops, orc, synth, rows, k, ntok):
    """The tile form of the f32 matvec: every output is the same -0.0-seeded left-to-right sum."""
    w = synth.normal_f32(rows * k, 5, "mm.w", rows, k, std=0.02).reshape(rows, k)
    x = synth.normal_f32(ntok * k, 5, "mm.x", rows, k).reshape(ntok, k)
    got = ops.matmul_f32_tokens(w, x)
    want = np.stack([orc.matvec_dequant(orc.F32, w, x[t], k, rows) for t in range(ntok)])
    assert bit_equal(got, want)
    z = ops.matmul_f32_tokens(-np.abs(w), np.zeros_like(x))
    assert np.all(np.signbit(z)), "an all -0.0 sum keeps its sign: no padding term enters a chain"


def test_silu_mul_and_quant(ops, orc, synth):
    g = synth.normal_f32(8 * 768, 6, "g") * np.float32(3.0)
    u = synth.normal_f32(8 * 768, 6, "u")
    want = orc.mul(orc.silu(g), u)
    got = ops.silu_mul(g, u)
    assert max_dev(got, want) <= ATTENTION
    ulp = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
    assert ulp.max() <= 2 and np.mean(ulp > 0) < 0.01, "exp differs from the host libm by at most an ulp, rarely"
    out, qs, d = ops.silu_mul_quant(g, u)
    assert bit_equal(out, got)
    hq, hd, _ = orc.quantize_q8k(got)  # the quantizer itself is exact on the device's own activations
    assert np.array_equal(qs, hq) and bit_equal(d, hd)
    # crates/llamd-cpu/src/lib.rs:282-290
    s = ops.silu_mul([0.0, 1.0, -1.0], [1.0, 1.0, 1.0])
    assert s[0] == 0.0 and abs(s[1] - 1.0 / (1.0 + np.exp(-1.0))) < F32_ULP * 2 and -1.0 < s[2] < 0.0


def test_moe_combine_is_bit_exact(ops, orc, synth):
    nseq, nu, E = 2, 8, 2048
    down = synth.normal_f32(nseq * nu * E, 7, "down").reshape(nseq, nu, E)
    w = np.abs(synth.normal_f32(nseq * nu, 7, "cw")).reshape(nseq, nu)
    res = synth.normal_f32(nseq * E, 7, "res").reshape(nseq, E)
    want = np.zeros((nseq, E), np.float32)
    for s in range(nseq):
        acc = np.zeros(E, np.float32)
        for e in range(nu):
            acc = (acc + (w[s, e] * down[s, e]).astype(np.float32)).astype(np.float32)
        want[s] = res[s] + acc
    assert bit_equal(ops.moe_combine_add(down, w, res), want)


def test_argmax_lowest_index_on_ties(ops, orc, synth):
    x = synth.normal_f32(2 * 151936, 8, "amax").reshape(2, 151936)
    x[0, 777] = x[0, 150000] = 9.0
    x[1, 151935] = 12.0
    assert ops.argmax(x).tolist() == [777, 151935]
    assert ops.argmax(np.zeros(1000, np.float32)).tolist() == [0]
    assert ops.argmax(x[0])[0] == orc.argmax(x[0])


def test_moe_group_is_a_stable_counting_sort(ops, synth):
    n_expert, n_used, nseq = 128, 8, 37
    rng = np.random.default_rng(9)
    ids = np.stack([rng.permutation(n_expert)[:n_used] for _ in range(nseq)]).astype(np.int32)
    g = ops.moe_group(ids, n_expert, n_used)
    flat = ids.ravel()
    assert g["gcount"].tolist() == np.bincount(flat, minlength=n_expert).tolist()
    assert g["gstart"].tolist() == (np.cumsum(g["gcount"]) - g["gcount"]).tolist()
    order = np.argsort(flat, kind="stable")
    assert g["pslot"].tolist() == order.tolist(), "pairs of an expert in ascending pair order"
    assert g["ptoken"].tolist() == (order // n_used).tolist()
    covered = []
    for e, first, cnt in g["work"].tolist():
        assert 1 <= cnt <= 8 and g["gstart"][e] <= first and first + cnt <= g["gstart"][e] + g["gcount"][e]
        covered.extend(range(first, first + cnt))
    assert covered == list(range(flat.size)), "the work list covers every pair once"
    empty = ops.moe_group(np.zeros((0, n_used), np.int32), n_expert, n_used)
    assert not empty["gcount"].any() and empty["work"].shape[0] == 0


@pytest.mark.parametrize("n_expert,n_used,nseq,hot", [
    (128, 8, 512, None),    # a full prefill tile
    (128, 8, 5120, None),   # the largest tile one launch takes: 40960 pairs
    (1024, 2, 33, None),    # the most experts, most of them empty
    (8, 1, 1, None),        # a single pair
    (16, 4, 300, 5),        # every token also picks expert 5: one group far longer than a warp's chunk
])
def test_moe_group_edges(ops, n_expert, n_used, nseq, hot):
    rng = np.random.default_rng(n_expert + nseq)
    ids = np.stack([rng.permutation(n_expert)[:n_used] for _ in range(nseq)]).astype(np.int32)
    if hot is not None:
        ids[:, 0] = hot
    g = ops.moe_group(ids, n_expert, n_used)
    flat = ids.ravel()
    order = np.argsort(flat, kind="stable")
    assert g["gcount"].tolist() == np.bincount(flat, minlength=n_expert).tolist()
    assert g["gstart"].tolist() == (np.cumsum(g["gcount"]) - g["gcount"]).tolist()
    assert np.array_equal(g["pslot"], order) and np.array_equal(g["ptoken"], order // n_used)
    work = g["work"]
    assert work.shape[0] == int(np.sum((g["gcount"] + 7) // 8))
    assert int(work[:, 2].sum()) == flat.size and work[:, 2].min() >= 1 and work[:, 2].max() <= 8


def test_embed_is_a_dequantized_row(ops, orc, synth):
    from llamd_rs_b200 import backend

    rows, blocks = 50, 3
    w = synth.q6k_blocks(rows * blocks, 10, "embd")
    t = backend.DeviceWeights.upload(w, rows, blocks)
    full = orc.dequantize(orc.Q6K, w, rows * blocks * 256).reshape(rows, blocks * 256)
    for tok in (0, 17, 49):
        assert bit_equal(ops.embed(t, tok), full[tok])
    with pytest.raises(backend.Malformed):
        ops.embed(t, 50)


@pytest.mark.parametrize("nseq", [1, 3])
def test_gate_up_with_the_silu_quant_tail(ops, orc, synth, nseq):
    """The slot's last CTA produces silu(gate)*up and its Q8_K form: same bits as the two separate launches."""
    from llamd_rs_b200 import backend

    n_expert, rows, k, n_used = 10, 512, 512, 4
    wa = synth.q6k_blocks(n_expert * rows * k // 256, 94, "tail.a")
    wb = synth.q6k_blocks(n_expert * rows * k // 256, 94, "tail.b")
    da = backend.DeviceWeights.upload(wa, n_expert * rows, k // 256)
    db = backend.DeviceWeights.upload(wb, n_expert * rows, k // 256)
    rng = np.random.default_rng(nseq)
    ids = np.stack([rng.permutation(n_expert)[:n_used] for _ in range(nseq)]).astype(np.int32)
    x = synth.normal_f32(nseq * k, 94, "tail.x", nseq).reshape(nseq, k)
    for _ in range(2):  # twice: the counters must be reusable
        got = ops.matvec_grouped_x2_silu_quant(da, db, ids, x, rows)
    want = ops.matvec_grouped_x2_silu_quant(da, db, ids, x, rows, fused=False)
    assert bit_equal(got[0], want[0]) and bit_equal(got[1], want[1])
    assert np.array_equal(got[2], want[2]) and bit_equal(got[3], want[3])


def test_attention_with_the_quantize_tail(ops, synth):
    n_head, n_head_kv, hd, max_kv = 8, 2, 64, 48
    pos = np.array([5, 47, 0], dtype=np.int32)
    kvd = n_head_kv * hd
    q = synth.normal_f32(3 * n_head * hd, 95, "atq.q")
    k = synth.normal_f32(3 * max_kv * kvd, 95, "atq.k")
    v = synth.normal_f32(3 * max_kv * kvd, 95, "atq.v")
    for _ in range(2):
        got = ops.attention_meta_quant(q, k, v, pos, n_head, n_head_kv, hd, max_kv)
    want = ops.attention_meta_quant(q, k, v, pos, n_head, n_head_kv, hd, max_kv, fused=False)
    assert bit_equal(got[0], want[0]) and np.array_equal(got[1], want[1]) and bit_equal(got[2], want[2])
