"""Full-size checks: the 48-layer, 128-expert Q6_K model of the decode benchmark.

The CUDA model and the CPU oracle decode the same seeded random-init weights.
Every routed expert id of every layer and every greedy token id must be equal
(EXACT); logits are held to tolerance::LOGITS (2e-3, tolerance.rs:109). The
oracle regenerates expert weights on demand, so 24 GB never sit on the host.
Size-independent properties cover the rest of the path at full size: graph
replay == plain queueing, the resident decode loop == forward() fed back.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
LOGITS = 2e-3


def max_dev(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.maximum(np.abs(a), np.abs(b)), 1.0)))


@pytest.fixture(scope="module")
def full():
    from llamd_rs_b200 import backend, synth
    from llamd_rs_b200.model import CudaModel

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    hp = dict(synth.QWEN3MOE_30B)
    m = CudaModel.load_synthetic(hp, 0, max_kv=96, max_seq=1)
    yield hp, m
    m.free()


def test_full_model_matches_the_oracle_token_for_token(full):
    import os

    import oracle
    from llamd_rs_b200 import synth

    hp, gm = full
    seed = 0
    w = dict(tok_embd=synth.q6k_blocks(hp["n_vocab"] * hp["n_embd"] // 256, seed, "tok_embd"),
             output_norm=np.ones(hp["n_embd"], np.float32),
             output=synth.q6k_blocks(hp["n_vocab"] * hp["n_embd"] // 256, seed, "output"),
             layers=[synth.layer_weights(hp, seed, il, with_experts=False) for il in range(hp["n_layer"])])
    om = oracle.Model(hp, w, threads=os.cpu_count() or 1,
                      expert_fn=lambda il, which, e: synth.expert_blocks(hp, seed, il, which, e))
    om.kv_new(8)
    prompt = synth.token_ids(2, hp["n_vocab"], 0, "prompt").tolist()
    gm.set_trace(True)
    tok_o = tok_g = None
    for pos in range(3):
        t_o = prompt[pos] if pos < len(prompt) else tok_o
        t_g = prompt[pos] if pos < len(prompt) else tok_g
        # oracle, layer by layer, to get the routing of every layer
        x = oracle.dequantize(oracle.Q6K, w["tok_embd"][t_o * (hp["n_embd"] // 256) * 210:], hp["n_embd"])
        ids_o = []
        for il in range(hp["n_layer"]):
            x, tr = om.forward_layer(il, x, pos)
            ids_o.append(tr["experts"].tolist())
        normed = oracle.mul(oracle.rms_norm(x, hp["rms_eps"]), w["output_norm"])
        logits_o = oracle.matvec_q6k(w["output"], normed, hp["n_embd"], hp["n_vocab"], threads=os.cpu_count() or 1)
        tok_o = oracle.argmax(logits_o)
        tok_g = gm.forward(t_g, pos)
        gx, gids = gm.read_trace()
        assert gids[:, 0, :].tolist() == ids_o, f"position {pos}: routed experts differ"
        assert max_dev(gm.logits()[0], logits_o) <= LOGITS, f"position {pos}: logits"
        assert tok_g == tok_o, f"position {pos}: greedy token gpu {tok_g} cpu {tok_o}"
    gm.set_trace(False)


def test_full_model_graph_and_resident_loop_agree_with_forward(full):
    from llamd_rs_b200 import synth

    hp, gm = full
    prompt = synth.token_ids(8, hp["n_vocab"], 1, "prompt").tolist()
    gm.use_graph = False
    for pos, t in enumerate(prompt):
        tok = gm.forward(t, pos)
    plain = [tok]
    for i in range(6):
        plain.append(gm.forward(plain[-1], len(prompt) + i))
    logits_plain = gm.logits()[0].copy()
    gm.use_graph = True
    for pos, t in enumerate(prompt):
        tok = gm.forward(t, pos)
    assert tok == plain[0]
    looped, ms = gm.decode(tok, len(prompt), 6)
    assert looped.tolist() == plain[1:], "resident loop == forward() fed back == un-graphed queueing"
    assert np.array_equal(gm.logits()[0].view(np.uint32), logits_plain.view(np.uint32))
    assert ms > 0


def test_full_model_prefill_equals_sequential_decode(full):
    """The tiled prefill (expert-major experts, 8 tokens per weight pass) against token-by-token decode."""
    from llamd_rs_b200 import synth

    hp, gm = full
    prompt = synth.token_ids(40, hp["n_vocab"], 2, "prefill").tolist()
    for pos, t in enumerate(prompt):
        tok = gm.forward(t, pos)
    logits = gm.logits()[0].copy()
    for tile in (16, 512):
        gm.prefill_tile = tile
        assert gm.prefill(prompt, 0) == tok
        assert np.array_equal(gm.logits()[0].view(np.uint32), logits.view(np.uint32)), f"tile {tile}"
    # with the expert matrices folded once and kept (nb = 8 and nb = 3 images at the benchmark's widths)
    gm.set_option("prefill_prefold", 1)
    for tile in (16, 512):
        gm.prefill_tile = tile
        assert gm.prefill(prompt, 0) == tok
        assert np.array_equal(gm.logits()[0].view(np.uint32), logits.view(np.uint32)), f"prefold, tile {tile}"
    gm.set_option("prefill_prefold", 0)
    gm.prefill_tile = 512
