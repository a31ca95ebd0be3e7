"""The resident decode kernel (one cooperative launch per token, grid barriers between a layer's phases) against the
per-op pass. Both walk the same arithmetic in the same order, so everything must be equal bit for bit: the hidden state
after every layer, the routed experts of every layer, the KV cache, the logits and the tokens; with plain launches,
with the captured graph and in the device-side decode loop."""
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


def run_traced(m, tokens_in, n_gen):
    """Feed tokens_in, then n_gen greedy tokens; -> (tokens, per-position (x trace, ids trace), logits of the last pass)."""
    m.set_trace(True)
    toks, traces, tok = [], [], None
    for pos in range(len(tokens_in) + n_gen):
        tok = m.forward(tokens_in[pos] if pos < len(tokens_in) else tok, pos)
        toks.append(tok)
        x, ids = m.read_trace()
        traces.append((x.copy(), ids.copy()))
    m.set_trace(False)
    return toks, traces, m.logits()[0].copy()


DIMS = {
    "tiny": None,  # synth.TINY
    "wider": dict(n_layer=3, n_embd=512, n_head=8, n_head_kv=2, head_dim=64, n_expert=16, n_expert_used=4, n_ff_expert=512, n_vocab=1024,
                  rope_freq_base=1e7, rms_eps=1e-6),
    "full3": "full",  # three layers of the benchmark's dimensions
}


@pytest.mark.parametrize("which", ["tiny", "wider", "full3"])
def test_resident_pass_equals_the_per_op_pass(be, which):
    from llamd_rs_b200 import synth
    from llamd_rs_b200.model import CudaModel

    hp = synth.TINY if which == "tiny" else (dict(synth.QWEN3MOE_30B, n_layer=3) if which == "full3" else DIMS[which])
    n_prompt, n_gen = 9, 8
    prompt = synth.token_ids(n_prompt, hp["n_vocab"], 21, "resident", which).tolist()
    m = CudaModel.load_synthetic(hp, 7, max_kv=64)
    try:
        want_toks, want_tr, want_logits = run_traced(m, prompt, n_gen)
        want_kv = [m.read_kv(il, n_prompt + n_gen) for il in range(hp["n_layer"])]
        m.set_option("resident", 1)
        got_toks, got_tr, got_logits = run_traced(m, prompt, n_gen)
        for pos, ((wx, wi), (gx, gi)) in enumerate(zip(want_tr, got_tr)):
            for il in range(hp["n_layer"]):
                assert gi[il].tolist() == wi[il].tolist(), f"position {pos} layer {il}: routed experts {gi[il].tolist()} vs {wi[il].tolist()}"
                bad = np.flatnonzero(bits(gx[il]).ravel() != bits(wx[il]).ravel())
                assert bad.size == 0, f"position {pos} layer {il}: {bad.size} of {gx[il].size} hidden values differ, first at {bad[0]}"
        assert got_toks == want_toks
        assert np.array_equal(bits(got_logits), bits(want_logits))
        for il in range(hp["n_layer"]):
            k, v = m.read_kv(il, n_prompt + n_gen)
            assert np.array_equal(bits(k), bits(want_kv[il][0])) and np.array_equal(bits(v), bits(want_kv[il][1])), f"KV cache of layer {il}"
        # the captured graph and the device-side loop
        m.use_graph = True
        tok = None
        for pos in range(n_prompt):
            tok = m.forward(prompt[pos], pos)
        assert tok == want_toks[n_prompt - 1]
        looped, ms = m.decode(tok, n_prompt, n_gen)
        assert looped.tolist() == want_toks[n_prompt:], "resident kernel inside the replayed graph"
        assert np.array_equal(bits(m.logits()[0]), bits(want_logits))
        assert m.launches_per_pass() < 12, "one resident launch, the head and the bookkeeping"
    finally:
        m.free()


LAYER = 1e-4   # crates/llamd-core/src/tolerance.rs:100
LOGITS = 2e-3  # tolerance.rs:109


def dev_rms(a, b):
    """Largest |a - b| relative to the rms of the exact vector. The reference's tolerances are stated for activations of
    order 1; the random-init models here carry hidden states of rms 50..500, so the deviation is scaled by the vector's own
    size instead of llamd_core::tolerance::max_deviation's floor of 1."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / max(float(np.sqrt(np.mean(b * b))), 1e-30))


@pytest.mark.parametrize("resident", [1, 0])
@pytest.mark.parametrize("which", ["tiny", "wider", "full3"])
def test_fast_arithmetic_is_the_same_function_up_to_rounding(be, which, resident):
    """Option arith = 1: reduction trees for the norms' sums, the router's dots and attention's sums, nothing else changed; in
    the resident kernel and in the graph of separate launches alike. Checked where rounding noise is all that can differ: at position 0 (softmax over one key is exactly 1) the hidden
    state after every layer stays within LAYER, the K/V rows within LAYER and the logits within LOGITS of the exact
    mode's, relative to each vector's rms, and the routed experts are the same. Later positions are only required to run
    and to be reproducible: a random-init network is chaotic (one flipped Q8_K rounding after a one-ulp change of a norm's
    scale moves a V row by 0.6 %, saturated softmaxes amplify that), so the modes' continuations drift apart there, which
    is why the exact mode is the default."""
    from llamd_rs_b200 import backend, synth
    from llamd_rs_b200.model import CudaModel

    hp = synth.TINY if which == "tiny" else (dict(synth.QWEN3MOE_30B, n_layer=3) if which == "full3" else DIMS[which])
    tokens = synth.token_ids(6, hp["n_vocab"], 33, "fast", which).tolist()
    m = CudaModel.load_synthetic(hp, 7, max_kv=64)
    try:
        m.set_option("resident", resident)
        _, exact_tr, _ = run_traced(m, tokens[:1], 0)
        exact_logits = m.logits()[0].copy()
        exact_kv = [m.read_kv(il, 1) for il in range(hp["n_layer"])]
        for mask in (2, 4, 8, 1):  # norms, router, attention, all
            m.set_option("arith", mask)
            _, fast_tr, _ = run_traced(m, tokens[:1], 0)
            fast_logits = m.logits()[0].copy()
            (ex, ei), (fx, fi) = exact_tr[0], fast_tr[0]
            assert np.array_equal(ei, fi), f"{which} mask {mask}: expert ids at position 0"
            for il in range(hp["n_layer"]):
                assert dev_rms(fx[il, 0], ex[il, 0]) <= LAYER, f"{which} mask {mask}: layer {il} hidden state"
                k, v = m.read_kv(il, 1)
                assert dev_rms(k, exact_kv[il][0]) <= LAYER and dev_rms(v, exact_kv[il][1]) <= LAYER, f"{which} mask {mask}: layer {il} K/V"
            assert dev_rms(fast_logits, exact_logits) <= LOGITS
        assert not np.array_equal(bits(fast_tr[0][0]), bits(exact_tr[0][0])), "the two modes should not be the same code path"
        with pytest.raises(backend.Malformed):
            m.set_option("arith", 3)
        # reproducible: the trees have a fixed shape
        toks_a, tr_a, log_a = run_traced(m, tokens, 4)
        toks_b, tr_b, log_b = run_traced(m, tokens, 4)
        assert toks_a == toks_b and np.array_equal(bits(log_a), bits(log_b))
        assert all(0 <= t < hp["n_vocab"] for t in toks_a)
        m.set_option("arith", 0)
        _, again_tr, _ = run_traced(m, tokens[:1], 0)
        assert np.array_equal(bits(again_tr[0][0]), bits(exact_tr[0][0])), "switching back restores the exact arithmetic"
    finally:
        m.free()


def test_fast_arithmetic_in_a_batch_of_sequences(be):
    """The graph of separate launches carries the tree sums for batches too: four sequences in one pass give what four
    single passes give in the same mode, bit for bit (the trees do not depend on the batch)."""
    from llamd_rs_b200 import synth
    from llamd_rs_b200.model import CudaModel

    hp = synth.TINY
    m = CudaModel.load_synthetic(hp, 7, max_kv=32, max_seq=4)
    try:
        m.set_option("arith", 1)
        toks = synth.token_ids(12, hp["n_vocab"], 4, "fast.batch").reshape(3, 4)
        single = []
        for s_ in range(4):
            for pos in range(3):
                t = m.forward(int(toks[pos, s_]), pos)
            single.append((t, m.logits()[0].copy()))
        for pos in range(3):
            out = m.forward_batch(toks[pos].tolist(), [pos] * 4)
        lb = m.logits(4)
        for s_ in range(4):
            assert int(out[s_]) == single[s_][0] and np.array_equal(bits(lb[s_]), bits(single[s_][1])), f"sequence {s_}"
    finally:
        m.free()
