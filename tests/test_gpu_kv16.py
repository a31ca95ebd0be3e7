"""The binary16 K/V cache (model option kv_f16; the benchmark configuration's "KV cache is f16").

The reference's caches are f32 (crates/llamd-runtime/src/kv.rs:27-170), so the oracle for this option is the oracle's
own f16-store mode: every appended K/V value rounded to binary16, nearest-even, the arithmetic otherwise unchanged.
Against it the GPU must give the same tokens, the same routed experts at every layer, and bit-identical cache rows;
and under the option every path of the model must agree with every other bit for bit, as they do over an f32 cache."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LOGITS = 2e-3  # crates/llamd-core/src/tolerance.rs:109


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def max_dev(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.maximum(np.abs(a), np.abs(b)), 1.0)))


@pytest.fixture(scope="module")
def be():
    from llamd_rs_b200 import backend

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    backend.stream_init()
    return backend


def test_decode_over_an_f16_cache_matches_the_oracles_f16_store_mode(be):
    import oracle
    from llamd_rs_b200 import synth
    from llamd_rs_b200.model import CudaModel

    hp = synth.TINY
    w = synth.make_model(hp, seed=7)
    gm = CudaModel.load_batched(hp, w, max_kv=64, max_seq=1)
    om = oracle.Model(hp, w, threads=4)
    try:
        gm.set_option("kv_f16", 1)
        om.kv_new(64, f16=True)
        prompt = synth.token_ids(6, hp["n_vocab"], 3, "kv16").tolist()
        gm.set_trace(True)
        tok_g = tok_o = None
        for pos in range(20):
            t_g = prompt[pos] if pos < len(prompt) else tok_g
            t_o = prompt[pos] if pos < len(prompt) else tok_o
            # the oracle layer by layer (appends to its f16-store cache), with the routed experts of every layer
            x = oracle.dequantize(oracle.Q6K, w["tok_embd"][t_o * hp["n_embd"] // 256 * 210:], hp["n_embd"])
            want_ids = []
            for il in range(hp["n_layer"]):
                x, tr = om.forward_layer(il, x, pos)
                want_ids.append(tr["experts"].tolist())
            lo = om.forward(t_o, pos)  # (the whole pass: rewrites this position's cache rows with the same values)
            tok_g = gm.forward(t_g, pos)
            _, gids = gm.read_trace()
            assert [gids[il, 0].tolist() for il in range(hp["n_layer"])] == want_ids, f"position {pos}: expert ids"
            tok_o = oracle.argmax(lo)
            assert tok_g == tok_o, f"position {pos}"
            assert max_dev(gm.logits()[0], lo) <= LOGITS
        n = 20
        for il in range(hp["n_layer"]):
            gk, gv = gm.read_kv(il, n)
            ok, ov = om.kv_layer(il, n)
            assert np.array_equal(bits(gk), bits(ok)) and np.array_equal(bits(gv), bits(ov)), f"layer {il}: cache rows"
            # and they ARE binary16 values
            assert np.array_equal(bits(gk), bits(gk.astype(np.float16).astype(np.float32)))
    finally:
        gm.free()


@pytest.mark.parametrize("which", ["tiny", "full3"])
def test_every_path_agrees_over_an_f16_cache(be, which):
    """Per-op decode (plain and graph), the device decode loop, the resident kernel, the tiled prefill (integer GEMM and
    dp4a, several tiles) and a wide batch: the same tokens, logits and cache rows, bit for bit."""
    from llamd_rs_b200 import synth
    from llamd_rs_b200.model import CudaModel

    hp = synth.TINY if which == "tiny" else dict(synth.QWEN3MOE_30B, n_layer=3)
    n_seq = 10
    m = CudaModel.load_synthetic(hp, 7, max_kv=64, max_seq=n_seq)
    try:
        m.set_option("kv_f16", 1)
        prompt = synth.token_ids(21, hp["n_vocab"], 5, "kv16.paths", which).tolist()
        seq_tok, seq_logits = {}, {}
        for pos, t in enumerate(prompt):
            seq_tok[pos + 1] = m.forward(t, pos)
            seq_logits[pos + 1] = m.logits()[0].copy()
        kv_ref = [m.read_kv(il, len(prompt)) for il in range(hp["n_layer"])]
        m.use_graph = False
        assert [m.forward(t, pos) for pos, t in enumerate(prompt)][-1] == seq_tok[len(prompt)]
        assert np.array_equal(bits(m.logits()[0]), bits(seq_logits[len(prompt)]))
        m.use_graph = True
        for tile, length in [(4, 5), (8, 17), (16, 21), (512, 21)]:
            m.prefill_tile = tile
            for gemm in (True, False):
                m.set_prefill_gemm(gemm)
                assert m.prefill(prompt[:length], 0) == seq_tok[length], f"tile {tile} length {length}"
                assert np.array_equal(bits(m.logits()[0]), bits(seq_logits[length])), f"tile {tile} length {length}: logits"
        m.set_prefill_gemm(True)
        m.prefill_tile = 512
        m.prefill(prompt, 0)
        for il in range(hp["n_layer"]):
            k, v = m.read_kv(il, len(prompt))
            assert np.array_equal(bits(k), bits(kv_ref[il][0])) and np.array_equal(bits(v), bits(kv_ref[il][1]))
        # greedy continuation: forward(), the device loop, the resident kernel
        tok0 = seq_tok[len(prompt)]
        want, tok = [], tok0
        for i in range(6):
            tok = m.forward(tok, len(prompt) + i)
            want.append(tok)
        got, _ = m.decode(tok0, len(prompt), 6)
        assert got.tolist() == want
        m.set_option("resident", 1)
        got, _ = m.decode(tok0, len(prompt), 6)
        assert got.tolist() == want
        tok, res = tok0, []
        for i in range(6):
            tok = m.forward(tok, len(prompt) + i)
            res.append(tok)
        assert res == want
        m.set_option("resident", 0)
        # a wide batch: every sequence gets the single-sequence pass's bits
        toks = synth.token_ids(n_seq * 3, hp["n_vocab"], 6, "kv16.batch", which).reshape(3, n_seq)
        single = []
        for s in range(n_seq):
            for pos in range(3):
                t = m.forward(int(toks[pos, s]), pos)
            single.append((t, m.logits()[0].copy()))
        for pos in range(3):
            out = m.forward_batch(toks[pos].tolist(), [pos] * n_seq)
        lb = m.logits(n_seq)
        for s in range(n_seq):
            assert int(out[s]) == single[s][0] and np.array_equal(bits(lb[s]), bits(single[s][1])), f"sequence {s}"
        # back to f32: a fresh, empty cache and the f32 results
        m.set_option("kv_f16", 0)
        f32_tok = [m.forward(t, pos) for pos, t in enumerate(prompt)][-1]
        k32, _ = m.read_kv(0, len(prompt))
        assert not np.array_equal(bits(k32), bits(kv_ref[0][0])), "an f32 cache keeps what binary16 would round away"
        assert 0 <= f32_tok < hp["n_vocab"]
    finally:
        m.free()
