"""Model::open + DeviceModel::load_batched from a GGUF file (crates/llamd-models/src/model.rs:108-131,
crates/llamd-runtime/src/device.rs:225-471) against the same weights handed over tensor by tensor: the file path must
change nothing, bit for bit, and must refuse what the reference refuses before any upload."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(tmp_path_factory):
    from llamd_rs_b200 import backend, gguf, synth
    from llamd_rs_b200.model import CudaModel

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    backend.stream_init()
    d = tmp_path_factory.mktemp("gguf")
    hp = dict(synth.TINY)
    path = d / "tiny.gguf"
    gguf.write_synthetic(path, hp, 7)
    return dict(be=backend, gg=gguf, synth=synth, M=CudaModel, hp=hp, path=path, dir=d)


def run(m, prompt, n_new=6):
    toks, t = [], None
    for pos, tok in enumerate(prompt):
        t = m.forward(tok, pos)
    toks.append(t)
    for i in range(n_new):
        t = m.forward(t, len(prompt) + i)
        toks.append(t)
    return toks, m.logits()[0].copy()


def test_file_model_equals_tensor_by_tensor_model(env):
    hp, synth = env["hp"], env["synth"]
    prompt = synth.token_ids(9, hp["n_vocab"], 3, "gguf").tolist()
    ref = env["M"].load_synthetic(hp, 7, max_kv=32)
    want_toks, want_logits = run(ref, prompt)
    want_bytes = ref.weight_bytes()
    ref.free()
    m = env["M"].open_gguf(env["path"], max_kv=32)
    assert m.hparams() == {k: (pytest.approx(v) if isinstance(v, float) else v) for k, v in hp.items()}
    assert m.weight_bytes() == want_bytes
    toks, logits = run(m, prompt)
    assert toks == want_toks
    assert np.array_equal(logits.view(np.uint32), want_logits.view(np.uint32)), "logits differ in some bit"
    # the file model prefills like any other
    assert m.prefill(prompt, 0) == want_toks[0]
    m.free()


def test_batched_file_model(env):
    hp, synth = env["hp"], env["synth"]
    m = env["M"].open_gguf(env["path"], max_kv=16, max_seq=4)
    one = env["M"].open_gguf(env["path"], max_kv=16)
    toks = synth.token_ids(4, hp["n_vocab"], 5, "gguf.b").tolist()
    got = m.forward_batch(toks, [0, 0, 0, 0]).tolist()
    assert got == [one.forward(t, 0) for t in toks]
    m.free(); one.free()


def rewritten(env, name, change):
    """The tiny model's tensor list with one entry replaced / removed by `change(list) -> list`."""
    gg, hp = env["gg"], env["hp"]
    with gg.Gguf.open(env["path"]) as g:
        ts = [(t.name, t.dims, t.ggml_type, g.tensor_data(t).copy()) for t in g.tensors]
    path = env["dir"] / name
    gg.write_gguf(path, gg.synthetic_metadata(hp), change(ts))
    return path


def test_f16_norms_and_tied_output(env):
    hp, synth, gg = env["hp"], env["synth"], env["gg"]
    prompt = synth.token_ids(5, hp["n_vocab"], 4, "gguf.t").tolist()

    def as_f16(ts):  # norm vectors stored as F16 (1.0 is exact): nothing may change
        return [(n, d, gg.GGML_F16, b.view(np.float32).astype(np.float16)) if n.endswith("_norm.weight") else (n, d, ty, b) for n, d, ty, b in ts]

    base = env["M"].open_gguf(env["path"], max_kv=16)
    want = run(base, prompt, 2)
    base.free()
    m = env["M"].open_gguf(rewritten(env, "f16.gguf", as_f16), max_kv=16)
    got = run(m, prompt, 2)
    m.free()
    assert got[0] == want[0] and np.array_equal(got[1], want[1])

    # no output.weight: the head reads the embedding table (model.rs:117-121)
    weights = synth.make_model(hp, 7)
    weights["output"] = None
    tied_ref = env["M"].load(hp, weights, max_kv=16)
    want = run(tied_ref, prompt, 2)
    tied_ref.free()
    m = env["M"].open_gguf(rewritten(env, "tied.gguf", lambda ts: [t for t in ts if t[0] != "output.weight"]), max_kv=16)
    got = run(m, prompt, 2)
    m.free()
    assert got[0] == want[0] and np.array_equal(got[1], want[1])


def test_refusals_before_the_upload(env):
    be, gg, hp, synth = env["be"], env["gg"], env["hp"], env["synth"]
    E, kvd = hp["n_embd"], hp["n_head_kv"] * hp["head_dim"]

    def q8_k(ts):  # a K projection stored as Q8_0
        return [(n, d, gg.GGML_Q8_0, synth.q8_0_blocks(kvd * E // 32, 1, "q8")) if n == "blk.1.attn_k.weight" else (n, d, ty, b) for n, d, ty, b in ts]

    with pytest.raises(be.Unsupported, match="blk.1.attn_k.weight is Q8_0, not Q6_K"):
        env["M"].open_gguf(rewritten(env, "q8.gguf", q8_k), max_kv=16)

    def short_v(ts):  # V with half the rows the hyperparameters give it
        return [(n, [E, kvd // 2], ty, b[: b.size // 2]) if n == "blk.0.attn_v.weight" else (n, d, ty, b) for n, d, ty, b in ts]

    with pytest.raises(be.Malformed, match="blk.0.attn_v.weight"):
        env["M"].open_gguf(rewritten(env, "shape.gguf", short_v), max_kv=16)

    def long_norm(ts):
        return [(n, [E + 1], ty, np.ones(E + 1, np.float32)) if n == "blk.0.ffn_norm.weight" else (n, d, ty, b) for n, d, ty, b in ts]

    with pytest.raises(be.Malformed, match="blk.0.ffn_norm.weight has"):
        env["M"].open_gguf(rewritten(env, "norm.gguf", long_norm), max_kv=16)
    with pytest.raises(be.Malformed, match="tensors missing"):
        env["M"].open_gguf(rewritten(env, "gone.gguf", lambda ts: [t for t in ts if t[0] != "blk.1.ffn_up_exps.weight"]), max_kv=16)
    with pytest.raises(be.Malformed, match="max_kv of 0"):
        env["M"].open_gguf(env["path"], max_kv=0)
    with pytest.raises(be.Malformed, match="max_seq"):
        env["M"].open_gguf(env["path"], max_kv=16, max_seq=99)
