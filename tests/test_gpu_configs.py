"""Parity at the sizes the benchmark configurations name, against the CPU oracle.

  config 1  the six decode matvec shapes x {Q6_K, Q8_0} x batch 1/2/4/8, every row, bit-exact. The shapes pick
            every branch of the launch logic: the sequence-group split of small matrices at batch > 1, the
            CTA-per-32-rows and the thread-per-row Q8_0 kernels (lm_head is the one that selects the latter by size).
  config 2  one MoE FFN layer at full size (f32 router 128x2048, 128 SwiGLU experts of 768) at T = 1 through the
            decode kernels and at T = 512 through the scatter plan and the grouped expert GEMM. Expert ids, routing
            weights, gate/up rows, activations, down rows and the combined output are all bit-exact (the device's
            exponential is made identical to the host libm's expf, see test_gpu_expf.py).
  config 3  the 48-layer model over the benchmark's own run: the 512-token prompt and 256 greedy tokens, checked
            against tests/golden/decode_seed0.npz (written by the CPU oracle, see make_decode_golden.py): the
            routed experts of every layer at every position and every token id, EXACT.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decode_seed0.npz")
THREADS = os.cpu_count() or 1


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bit_equal(got, want, what=""):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    bad = np.flatnonzero(bits(got).ravel() != bits(want).ravel())
    assert bad.size == 0, f"{what}: {bad.size} of {got.size} differ, first at {bad[0]}: gpu {got.ravel()[bad[0]]!r} cpu {want.ravel()[bad[0]]!r}"


def max_dev(a, b):
    """tolerance::max_deviation: |a-b| / max(1, |a|, |b|)."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.maximum(np.abs(a), np.abs(b)), 1.0)))


@pytest.fixture(scope="module")
def be():
    from llamd_rs_b200 import backend

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    backend.stream_init()
    return backend


# ---- config 1 -----------------------------------------------------------------------------------------------
SHAPES = [("attn_q", 4096, 2048), ("attn_k", 512, 2048), ("attn_out", 2048, 4096), ("expert_gate", 768, 2048),
          ("expert_down", 2048, 768), ("lm_head", 151936, 2048)]


def oracle_q8_0_rows(orc, w, x, k, rows):
    """The dequantize-then-sequential-dot path, a slab of rows at a time (the oracle dequantizes what it is given whole)."""
    row_bytes = k // 32 * 34
    out = np.empty(rows, np.float32)
    for r0 in range(0, rows, 16384):
        r1 = min(rows, r0 + 16384)
        out[r0:r1] = orc.matvec_dequant(orc.Q8_0, w[r0 * row_bytes:r1 * row_bytes], x, k, r1 - r0, threads=THREADS)
    return out


@pytest.mark.parametrize("name,rows,k", SHAPES)
@pytest.mark.parametrize("ty", ["q6k", "q8_0"])
def test_config1_matvec_shapes_are_bit_exact(be, orc, name, rows, k, ty):
    from llamd_rs_b200 import synth

    x = synth.normal_f32(8 * k, 1, "config1.x", name)
    if ty == "q6k":
        w = synth.q6k_blocks(rows * k // 256, 0, "config1", name)
        dw = be.DeviceWeights.upload(w, rows, k // 256)
        want = [orc.matvec_q6k(w, x[s * k:(s + 1) * k], k, rows, threads=THREADS) for s in range(8)]
    else:
        w = synth.q8_0_blocks(rows * k // 32, 0, "config1", name)
        dw = be.Q80Weights.upload(w, rows, k // 32)
        want = [oracle_q8_0_rows(orc, w, x[s * k:(s + 1) * k], k, rows) for s in range(8)]
    for batch in (1, 2, 4, 8):
        got = dw.matvec_f32(x[:batch * k], batch)
        for s in range(batch):
            assert_bit_equal(got[s], want[s], f"{name} {ty} batch {batch} sequence {s}")
    dw.free()


# ---- config 2 -----------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def moe_layer(be):
    from llamd_rs_b200 import synth

    E, ffe, ne = 2048, 768, 128
    router = synth.normal_f32(ne * E, 0, "config2.router", std=0.02).reshape(ne, E)
    w = {n: synth.q6k_blocks(ne * ffe * E // 256, 0, "config2", n) for n in ("gate", "up", "down")}
    dev = {"gate": be.DeviceWeights.upload(w["gate"], ne * ffe, E // 256), "up": be.DeviceWeights.upload(w["up"], ne * ffe, E // 256),
           "down": be.DeviceWeights.upload(w["down"], ne * E, ffe // 256)}
    yield dict(E=E, ffe=ffe, ne=ne, nu=8, router=router, w=w, dev=dev, per=ffe * E // 256 * 210)
    for d in dev.values():
        d.free()


def oracle_moe_token(orc, L, x):
    """route + moe_ffn for one token on the CPU oracle -> dict of everything the device is compared with."""
    E, ffe, per = L["E"], L["ffe"], L["per"]
    logits = orc.matvec_dequant(orc.F32, L["router"], x, E, L["ne"])
    r = orc.route(logits, L["nu"])
    gate, up, act, down = [], [], [], []
    out = np.zeros(E, np.float32)
    for e, wt in zip(r["experts"], r["weights"]):
        e = int(e)
        g = orc.matvec_q6k(L["w"]["gate"][e * per:(e + 1) * per], x, E, ffe, threads=THREADS)
        u = orc.matvec_q6k(L["w"]["up"][e * per:(e + 1) * per], x, E, ffe, threads=THREADS)
        a = orc.mul(orc.silu(g), u)
        d = orc.matvec_q6k(L["w"]["down"][e * per:(e + 1) * per], a, ffe, E, threads=THREADS)
        out = (out + np.float32(wt) * d).astype(np.float32)  # one f32 multiply, one f32 add per element, in routing order
        gate.append(g), up.append(u), act.append(a), down.append(d)
    return dict(logits=logits, ids=r["experts"], weights=r["weights"], gate=np.stack(gate), up=np.stack(up), act=np.stack(act),
                down=np.stack(down), out=out)


def combine_in_order(down, weights):
    out = np.zeros(down.shape[1], np.float32)
    for e in range(down.shape[0]):
        out = (out + (np.float32(weights[e]) * down[e]).astype(np.float32)).astype(np.float32)
    return out


def test_config2_moe_layer_decode(be, orc, moe_layer):
    """T = 1: the decode kernels (router matvec + route, grouped gate/up, SiLU x up + Q8_K, per-slot down, ordered combine)."""
    from llamd_rs_b200 import ops, synth

    L = moe_layer
    for t in range(4):
        x = synth.normal_f32(L["E"], 0, "config2.x", t)
        o = oracle_moe_token(orc, L, x)
        logits, ids, wts = ops.router_matvec(L["router"], x[None], L["nu"])
        assert_bit_equal(logits[0], o["logits"], "router logits")
        assert ids[0].tolist() == o["ids"].tolist(), "routed experts, best first"
        assert_bit_equal(wts[0], o["weights"], "routing weights (the device's exp is the host libm's)")
        gate, up, q2, d2 = ops.matvec_grouped_x2_silu_quant(L["dev"]["gate"], L["dev"]["up"], ids, x[None], L["ffe"], fused=False)
        assert_bit_equal(gate, o["gate"], "gate rows")
        assert_bit_equal(up, o["up"], "up rows")
        act = ops.silu_mul(gate.ravel(), up.ravel()).reshape(L["nu"], L["ffe"])
        assert_bit_equal(act, o["act"], "silu(gate) * up")
        hq, hd, _ = orc.quantize_q8k(act.ravel())
        assert np.array_equal(q2.ravel(), hq) and np.array_equal(bits(d2.ravel()), bits(hd)), "Q8_K of the device's activation"
        down = ops.matvec_grouped_pa(L["dev"]["down"], ids[0], q2, d2, L["E"])
        for s, e in enumerate(ids[0]):
            want = orc.matvec_q6k_q8k(L["w"]["down"][int(e) * L["per"]:(int(e) + 1) * L["per"]], q2[s], d2[s], L["ffe"], L["E"], threads=THREADS)
            assert_bit_equal(down[s], want, f"down rows of slot {s}")
        out = ops.moe_combine_add(down[None], wts, None)[0]
        assert_bit_equal(out, combine_in_order(down, wts[0]), "combine in routing order")
        assert_bit_equal(down, o["down"], "down rows against the CPU path")
        assert_bit_equal(out, o["out"], "moe_ffn output against the CPU path")


def test_config2_moe_layer_prefill_512(be, orc, moe_layer):
    """T = 512: f32 router GEMM + route per token, the scatter plan, the grouped expert GEMM (integer tensor path)."""
    from llamd_rs_b200 import ops, synth

    L = moe_layer
    T, nu, E, ffe, per = 512, L["nu"], L["E"], L["ffe"], L["per"]
    x = synth.normal_f32(T * E, 0, "config2.x512").reshape(T, E)
    logits = ops.matmul_f32_tokens(L["router"], x)
    ids, wts, _ = ops.router(logits, nu)
    plan = ops.moe_group(ids, L["ne"], nu)
    assert int(plan["gcount"].sum()) == T * nu and sorted(plan["pslot"].tolist()) == list(range(T * nu))
    gate, up = ops.expert_major([L["dev"]["gate"], L["dev"]["up"]], x, ids, ffe, gemm=True)
    act = ops.silu_mul(gate.ravel(), up.ravel()).reshape(T * nu, ffe)
    (down,) = ops.expert_major([L["dev"]["down"]], act, ids, E, by_slot=True, gemm=True)
    out = ops.moe_combine_add(down.reshape(T, nu, E), wts, None)
    for t in range(T):
        o = oracle_moe_token(orc, L, x[t])
        assert_bit_equal(logits[t], o["logits"], f"token {t}: router logits")
        assert ids[t].tolist() == o["ids"].tolist(), f"token {t}: routed experts"
        assert_bit_equal(wts[t], o["weights"], f"token {t}: routing weights")
        assert_bit_equal(gate[t * nu:(t + 1) * nu], o["gate"], f"token {t}: gate rows")
        assert_bit_equal(up[t * nu:(t + 1) * nu], o["up"], f"token {t}: up rows")
        assert_bit_equal(act[t * nu:(t + 1) * nu], o["act"], f"token {t}: silu(gate) * up")
        assert_bit_equal(down[t * nu:(t + 1) * nu], o["down"], f"token {t}: down rows")
        assert_bit_equal(out[t], o["out"], f"token {t}: moe_ffn output")


# ---- config 3 -----------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def golden():
    if not os.path.exists(GOLDEN):
        pytest.fail("tests/golden/decode_seed0.npz is missing (python tests/golden/make_decode_golden.py writes it)")
    g = np.load(GOLDEN)
    return dict(prompt=g["prompt"], chosen=g["chosen"], experts=g["experts"], done=int(g["done"]))


def test_config3_decode_run_matches_the_cpu_path(be, golden):
    """Every routed expert of every layer at every position of the 512-token prompt and the greedy tokens after it,
    and every token id, against the CPU oracle's run of the same seeded model."""
    from llamd_rs_b200 import synth
    from llamd_rs_b200.model import CudaModel

    hp = dict(synth.QWEN3MOE_30B)
    n_prompt, n_pos = golden["prompt"].size, golden["done"]
    assert n_pos >= n_prompt + 32, "the golden run must cover at least 32 decoded positions"
    m = CudaModel.load_synthetic(hp, 0, max_kv=n_pos + 8, max_seq=1)
    try:
        # token by token with the per-layer trace: routed experts at every position, tokens from the last prompt position on
        m.set_trace(True)
        tok = None
        for pos in range(n_pos):
            t = int(golden["prompt"][pos]) if pos < n_prompt else tok
            tok = m.forward(t, pos)
            _, ids = m.read_trace()
            got = ids[:, 0, :].tolist()
            if got != golden["experts"][pos].tolist():
                il = next(i for i in range(hp["n_layer"]) if got[i] != golden["experts"][pos][i].tolist())
                pytest.fail(f"position {pos}, layer {il}: routed experts gpu {got[il]} cpu {golden['experts'][pos][il].tolist()}")
            if pos >= n_prompt - 1:
                assert tok == int(golden["chosen"][pos]), f"position {pos}: greedy token gpu {tok} cpu {int(golden['chosen'][pos])}"
        m.set_trace(False)
        # the tiled prefill: its token is the CPU path's
        assert m.prefill(golden["prompt"].tolist(), 0) == int(golden["chosen"][n_prompt - 1])
        # the resident loop (graph replay, token fed back on the device) over the decoded positions
        n_dec = n_pos - n_prompt
        toks, _ = m.decode(int(golden["chosen"][n_prompt - 1]), n_prompt, n_dec)
        assert toks.tolist() == golden["chosen"][n_prompt:n_pos].tolist(), "greedy tokens of the resident loop"
        # the same loop through the resident decode kernel (one cooperative launch per token)
        m.set_option("resident", 1)
        toks, _ = m.decode(int(golden["chosen"][n_prompt - 1]), n_prompt, n_dec)
        assert toks.tolist() == golden["chosen"][n_prompt:n_pos].tolist(), "greedy tokens of the resident decode kernel"
    finally:
        m.free()
