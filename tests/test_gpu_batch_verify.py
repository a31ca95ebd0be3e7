"""Wide batches and draft verification against single-sequence decode.

  - forward_batch with more than 8 sequences (the nseq kernels' limit per launch) runs either as the decode pass of matvec
    launches, whose large matrices then take one launch per 8 sequences (up to option matvec_batch_max sequences, 56 by
    default), or as a tile whose tokens belong to different sequences (beyond); either way every sequence must get
    exactly the tokens and logits of its own single-sequence run
    (crates/llamd-testing/tests/batch_decode.rs:102-125, beyond its 8);
  - verify() returns the greedy token after every prefix of what it is given, so speculative decoding with ANY drafter
    reproduces plain greedy decode token for token (the reference's rule for it: "acceptance may change speed; it may
    never change output", docs/porting-matrix.md row 20).
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


@pytest.mark.parametrize("path", ["matvec", "tile"])
@pytest.mark.parametrize("nseq", [9, 20, 33])
def test_wide_batch_equals_single_sequences(be, nseq, path):
    from llamd_rs_b200 import synth
    from llamd_rs_b200.model import CudaModel

    hp = synth.TINY
    steps = 5
    first = synth.token_ids(nseq, hp["n_vocab"], 31, "wide", nseq).tolist()
    single = CudaModel.load_synthetic(hp, 9, max_kv=16)
    want_toks, want_logits = [], []
    for s in range(nseq):
        tok, seq = first[s], []
        for pos in range(steps):
            tok = single.forward(tok, pos)
            seq.append(tok)
        want_toks.append(seq)
        want_logits.append(single.logits()[0].copy())
    single.free()
    m = CudaModel.load_synthetic(hp, 9, max_kv=16, max_seq=nseq)
    try:
        m.set_option("matvec_batch_max", 256 if path == "matvec" else 8)
        toks = np.array(first, dtype=np.int32)
        got = []
        for pos in range(steps):
            toks = m.forward_batch(toks, [pos] * nseq)
            got.append(toks.tolist())
        for s in range(nseq):
            assert [g[s] for g in got] == want_toks[s], f"sequence {s} of {nseq}"
        logits = m.logits(nseq)
        for s in range(nseq):
            assert np.array_equal(bits(logits[s]), bits(want_logits[s])), f"logits of sequence {s}"
        # sequences at different positions in one pass: restart every third sequence from position 0
        pos = [0 if s % 3 == 0 else steps for s in range(nseq)]
        toks2 = np.array([first[s] if s % 3 == 0 else got[-1][s] for s in range(nseq)], dtype=np.int32)
        out = m.forward_batch(toks2, pos)
        for s in range(0, nseq, 3):
            assert out[s] == want_toks[s][0]
        with pytest.raises(be.Malformed):
            m.forward_batch(np.zeros(nseq + 1, np.int32), [0] * (nseq + 1))
    finally:
        m.free()


def test_verify_and_speculative_decoding_reproduce_greedy_decode(be):
    from llamd_rs_b200 import synth
    from llamd_rs_b200.model import CudaModel

    hp = synth.TINY
    prompt = synth.token_ids(6, hp["n_vocab"], 41, "verify").tolist()
    n_gen = 24
    m = CudaModel.load_synthetic(hp, 9, max_kv=64)
    try:
        tok = m.prefill(prompt, 0)
        plain, _ = m.decode(tok, len(prompt), n_gen)
        plain = plain.tolist()
        full = prompt + [tok] + plain  # token i+1 is the greedy token after tokens[0..=i], from the end of the prompt on
        # verify: every prefix's greedy token, in tiles (prefill_tile 4 cuts these 20 tokens into five tiles)
        m.prefill_tile = 4
        got = m.verify(full[:20], 0)
        assert got[len(prompt) - 1:].tolist() == full[len(prompt):21]
        m.prefill_tile = 512
        assert m.verify(full[:20], 0).tolist() == got.tolist(), "the tile size changes nothing"
        # drafters: always right, always wrong, right then wrong; the output never changes, the number of passes does
        m.prefill(prompt, 0)
        oracle_draft = lambda out, k: plain[len(out) + 1:len(out) + 1 + k]
        spec, passes = m.speculative_decode(tok, len(prompt), n_gen, lambda out, k: plain[len(out):len(out) + k], max_draft=6)
        assert spec == plain and passes < n_gen / 3
        m.prefill(prompt, 0)
        spec, passes = m.speculative_decode(tok, len(prompt), n_gen, lambda out, k: [(t + 1) % hp["n_vocab"] for t in plain[len(out):len(out) + k]])
        assert spec == plain and passes == n_gen
        m.prefill(prompt, 0)
        half = lambda out, k: [t if i < 2 else (t + 7) % hp["n_vocab"] for i, t in enumerate(plain[len(out):len(out) + k])]
        spec, passes = m.speculative_decode(tok, len(prompt), n_gen, half, max_draft=5)
        assert spec == plain and n_gen / 4 < passes < n_gen
        # decoding goes on from the verified state exactly as from the plain one
        assert m.forward(plain[-1], len(prompt) + n_gen) == CudaModelRun(hp, prompt, n_gen + 1)[-1]
        del oracle_draft
    finally:
        m.free()


def CudaModelRun(hp, prompt, n_gen):
    from llamd_rs_b200.model import CudaModel

    m = CudaModel.load_synthetic(hp, 9, max_kv=64)
    try:
        tok = m.prefill(prompt, 0)
        out, _ = m.decode(tok, len(prompt), n_gen)
        return out.tolist()
    finally:
        m.free()
