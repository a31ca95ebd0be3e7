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
