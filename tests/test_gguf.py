"""The GGUF reader behind llamd_gguf.h, on CPU: what Gguf::parse accepts and refuses
(crates/llamd-gguf/src/lib.rs:124-213,290-376), tensor_data's checks (:231-256), Hparams::from_gguf
(crates/llamd-models/src/hparams.rs:78-175) and Model::verify_present (crates/llamd-models/src/model.rs:133-160).
The reference has no test file for its reader; the cases are its documented refusals, one each."""
import struct

import numpy as np
import pytest


@pytest.fixture(scope="module")
def gg():
    import __graft_entry__ as g

    g.build()
    from llamd_rs_b200 import gguf

    return gguf


@pytest.fixture(scope="module")
def be():
    from llamd_rs_b200 import backend

    return backend


@pytest.fixture(scope="module")
def synth():
    from llamd_rs_b200 import synth

    return synth


def gstr(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def header(n_tensors, n_kv, version=3, magic=b"GGUF"):
    return magic + struct.pack("<IQQ", version, n_tensors, n_kv)


def test_round_trip_of_every_value_type_and_tensor_type(gg, synth, tmp_path):
    q6 = synth.q6k_blocks(4, 1, "gguf.q6")
    q8 = synth.q8_0_blocks(3, 1, "gguf.q8")
    f32 = np.arange(5, dtype=np.float32)
    f16 = np.arange(7, dtype=np.float16)
    meta = {
        "general.architecture": "qwen3moe",
        "a.u8": gg.Typed(0, 200), "a.i8": gg.Typed(1, -3), "a.u16": gg.Typed(2, 60000), "a.i16": gg.Typed(3, 7),
        "a.u32": 123456, "a.i32": gg.Typed(5, -1), "a.f32": 1.5, "a.bool": True, "a.u64": 1 << 40, "a.i64": gg.Typed(11, 9),
        "a.f64": gg.Typed(12, 0.1), "a.list": [1, 2, 3], "a.strs": ["x", "yy"], "a.empty": gg.Typed(9, [], inner=8),
    }
    path = tmp_path / "t.gguf"
    size = gg.write_gguf(path, meta, [("w.q6", [256, 4], gg.GGML_Q6_K, q6), ("w.q8", [96], gg.GGML_Q8_0, q8),
                                      ("w.f32", [5], gg.GGML_F32, f32), ("w.f16", [7], gg.GGML_F16, f16)])
    with gg.Gguf.open(path) as g:
        assert (g.version, g.alignment, g.file_size()) == (3, 32, size)
        assert g.data_offset % 32 == 0
        assert g.keys() == sorted(meta), "metadata is kept sorted by key"
        assert g.architecture() == "qwen3moe"
        # Value::as_u64: every unsigned type, and signed ones when non-negative
        assert [g.get_u64(k) for k in ("a.u8", "a.u16", "a.u32", "a.u64", "a.i16", "a.i64")] == [200, 60000, 123456, 1 << 40, 7, 9]
        assert g.get_u64("a.i8") is None and g.get_u64("a.i32") is None, "negative values are not u64"
        assert g.get_u64("a.f32") is None and g.get_u64("a.bool") is None and g.get_u64("missing") is None
        # Value::as_f32: F32 as is, F64 rounded once
        assert g.get_f32("a.f32") == 1.5 and g.get_f32("a.f64") == float(np.float32(0.1)) and g.get_f32("a.u32") is None
        assert g.get_str("a.u32") is None
        assert [g.get_array_len(k) for k in ("a.list", "a.strs", "a.empty", "a.u8")] == [3, 2, 0, None]
        assert [t.name for t in g.tensors] == ["w.q6", "w.q8", "w.f32", "w.f16"]
        t = g.tensor("w.q6")
        assert (t.dims, t.ggml_type, t.elems(), t.offset) == ([256, 4], 14, 1024, 0)
        assert g.tensor("nope") is None
        assert np.array_equal(g.tensor_data(t), q6.view(np.uint8).ravel())
        assert np.array_equal(g.tensor_data(g.tensor("w.q8")), q8.view(np.uint8).ravel())
        assert np.array_equal(g.tensor_data(g.tensor("w.f32")).view(np.float32), f32)
        assert np.array_equal(g.tensor_data(g.tensor("w.f16")).view(np.float16), f16)
        assert all(x.offset % 32 == 0 for x in g.tensors)


def test_custom_alignment_moves_the_data_section(gg, tmp_path):
    path = tmp_path / "a.gguf"
    gg.write_gguf(path, {"k": 1}, [("t", [3], gg.GGML_F32, np.ones(3, np.float32)), ("u", [1], gg.GGML_F32, np.full(1, 2, np.float32))], alignment=256)
    with gg.Gguf.open(path) as g:
        assert g.alignment == 256 and g.data_offset % 256 == 0 and g.tensor("u").offset == 256
        assert g.tensor_data(g.tensor("u")).view(np.float32)[0] == 2


@pytest.mark.parametrize("blob,kind,needle", [
    (b"GGML" + struct.pack("<IQQ", 3, 0, 0), "Malformed", "magic"),
    (header(0, 0, version=2), "Unsupported", "version 2"),
    (b"GG", "Malformed", "truncated"),
    (b"", "Malformed", "truncated"),
    (header(0, 0)[:-3], "Malformed", "truncated"),
    (header(1 << 40, 0), "Malformed", "exceeds"),
    (header(0, 1 << 40), "Malformed", "exceeds"),
    (header(0, 1) + gstr("k") + struct.pack("<I", 13), "Malformed", "unknown type 13"),
    (header(0, 1) + gstr("k") + struct.pack("<IIQ", 9, 9, 0), "Unsupported", "nested"),
    (header(0, 1) + gstr("k") + struct.pack("<IIQ", 9, 4, 1 << 62), "Malformed", "elements declared"),
    (header(0, 1) + struct.pack("<Q", 1 << 50), "Malformed", "truncated"),
    (header(0, 1) + gstr("general.alignment") + struct.pack("<II", 4, 24), "Malformed", "power of two"),
    (header(0, 1) + gstr("general.alignment") + struct.pack("<II", 4, 0), "Malformed", "power of two"),
    (header(1, 0) + gstr("t") + struct.pack("<I", 5), "Malformed", "5 dimensions"),
    (header(1, 0) + gstr("t") + struct.pack("<IQ", 1, 4), "Malformed", "truncated"),
])
def test_parse_refusals(gg, be, blob, kind, needle):
    with pytest.raises(getattr(be, kind)) as e:
        gg.Gguf.parse(blob)
    assert needle in str(e.value)


def test_the_data_section_must_start_inside_the_file(gg, be):
    # 24 header bytes round up to offset 32, which is past the end of a 24-byte file
    with pytest.raises(be.Malformed, match="data section starts at 32"):
        gg.Gguf.parse(header(0, 0))
    g = gg.Gguf.parse(header(0, 0) + b"\0" * 8)
    assert g.tensors == [] and g.keys() == [] and g.data_offset == 32


def tinfo(name, dims, ty, off):
    return gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ty, off)


def padded(blob, extra=b""):
    return blob + b"\0" * ((-len(blob)) % 32) + extra


def test_tensor_data_refusals(gg, be):
    # extent past the end of the file
    g = gg.Gguf.parse(padded(header(1, 0) + tinfo("t", [8], 0, 0), b"\0" * 16))
    with pytest.raises(be.Malformed, match="past the"):
        g.tensor_data(g.tensor("t"))
    # a partial block: 100 elements of Q6_K
    g = gg.Gguf.parse(padded(header(1, 0) + tinfo("t", [100], 14, 0), b"\0" * 512))
    with pytest.raises(be.Malformed, match="not a multiple of the 256-element block"):
        g.tensor_data(g.tensor("t"))
    # a type the reader does not implement (Q4_K = 12)
    g = gg.Gguf.parse(padded(header(1, 0) + tinfo("t", [256], 12, 0), b"\0" * 512))
    with pytest.raises(be.Unsupported, match="type 12"):
        g.tensor_data(g.tensor("t"))
    # element count that overflows, offset that overflows
    g = gg.Gguf.parse(padded(header(2, 0) + tinfo("big", [1 << 40, 1 << 40], 0, 0) + tinfo("far", [1], 0, (1 << 64) - 8), b"\0" * 64))
    with pytest.raises(be.Malformed):
        g.tensor_data(g.tensor("big"))
    with pytest.raises(be.Malformed):
        g.tensor_data(g.tensor("far"))
    # zero-dimensional tensor: one element (an empty product)
    g = gg.Gguf.parse(padded(header(1, 0) + tinfo("s", [], 0, 0), struct.pack("<f", 3.0) + b"\0" * 28))
    assert g.tensor_data(g.tensor("s")).view(np.float32)[0] == 3.0


def test_open_reports_io_errors(gg, tmp_path):
    with pytest.raises(OSError):
        gg.Gguf.open(tmp_path / "absent.gguf")
    (tmp_path / "empty.gguf").write_bytes(b"")
    from llamd_rs_b200 import backend

    with pytest.raises(backend.Malformed, match="truncated"):
        gg.Gguf.open(tmp_path / "empty.gguf")


# ---- Hparams::from_gguf, verify_present -------------------------------------------------------------------------------
def tiny_file(gg, synth, tmp_path, name="tiny.gguf", drop_meta=(), meta_extra=None, drop_tensors=(), n_layer=None):
    hp = dict(synth.TINY)
    if n_layer:
        hp["n_layer"] = n_layer
    meta = gg.synthetic_metadata(hp)
    for k in drop_meta:
        del meta[k]
    meta.update(meta_extra or {})
    E = hp["n_embd"]
    kvd = hp["n_head_kv"] * hp["head_dim"]
    # header-only model: the tensor table is what from_gguf and verify_present look at, one small real tensor is enough
    names = ["token_embd.weight", "output_norm.weight", "output.weight"]
    for il in range(hp["n_layer"]):
        names += [f"blk.{il}.{s}.weight" for s in ("attn_norm", "attn_q", "attn_k", "attn_v", "attn_q_norm", "attn_k_norm", "attn_output",
                                                   "ffn_norm", "ffn_gate_inp", "ffn_gate_exps", "ffn_up_exps", "ffn_down_exps")]
    dims = {"token_embd.weight": [E, hp["n_vocab"]], "blk.0.attn_k.weight": [E, kvd]}
    ts = [(n, dims.get(n, [1]), gg.GGML_F32, None) for n in names if n not in drop_tensors]
    # write by hand: tensor infos that all point at one 4-byte payload (sizes are not checked until data is asked for)
    blob = bytearray(header(len(ts), len(meta)))
    for k, v in meta.items():
        t = v if isinstance(v, gg.Typed) else gg.Typed(gg._infer(v), v)
        blob += gstr(k) + struct.pack("<I", t.ty) + gg._value(t.ty, t.value, t.inner)
    for n, d, ty, _ in ts:
        blob += tinfo(n, d, ty, 0)
    path = tmp_path / name
    path.write_bytes(padded(bytes(blob), b"\0" * 32))
    return hp, path


def test_hparams_of_a_qwen3moe_file(gg, synth, tmp_path):
    hp, path = tiny_file(gg, synth, tmp_path)
    with gg.Gguf.open(path) as g:
        got = g.hparams()
        for k, v in hp.items():
            assert got[k] == (pytest.approx(v) if isinstance(v, float) else v), k
        assert (got["arch"], got["n_ff"], got["n_ctx_train"]) == ("qwen3moe", 5472, 262144)
        g.verify_present()


def test_head_dim_fallbacks(gg, synth, tmp_path):
    """key_length, else attn_k's output width over the kv heads, else n_embd / n_head (hparams.rs:106-117)."""
    p = "qwen3moe.attention.key_length"
    hp, path = tiny_file(gg, synth, tmp_path, "nokey.gguf", drop_meta=[p])
    with gg.Gguf.open(path) as g:
        assert g.hparams()["head_dim"] == hp["head_dim"], "from blk.0.attn_k.weight [n_embd, n_head_kv * head_dim]"
    hp, path = tiny_file(gg, synth, tmp_path, "nokey_nok.gguf", drop_meta=[p], drop_tensors=["blk.0.attn_k.weight"])
    with gg.Gguf.open(path) as g:
        assert g.hparams()["head_dim"] == hp["n_embd"] // hp["n_head"]


def test_hparams_refusals(gg, be, synth, tmp_path):
    cases = [
        (dict(meta_extra={"general.architecture": "llama"}), be.Unsupported, "llama; LLAMD implements qwen3 and qwen3moe"),
        (dict(drop_meta=["general.architecture"]), be.Malformed, "general.architecture is absent"),
        (dict(drop_meta=["qwen3moe.block_count"]), be.Malformed, "qwen3moe.block_count is absent"),
        (dict(drop_meta=["qwen3moe.expert_count"]), be.Malformed, "qwen3moe.expert_count is absent"),
        (dict(drop_meta=["qwen3moe.rope.freq_base"]), be.Malformed, "rope.freq_base is absent"),
        (dict(meta_extra={"qwen3moe.rope.freq_base": 10000}), be.Malformed, "rope.freq_base is absent"),  # an integer is not as_f32
        (dict(meta_extra={"qwen3moe.attention.head_count_kv": 3}), be.Malformed, "do not divide"),
        (dict(meta_extra={"qwen3moe.attention.head_count_kv": 0}), be.Malformed, "do not divide"),
        (dict(meta_extra={"qwen3moe.attention.key_length": 31}), be.Malformed, "must be even"),
        (dict(meta_extra={"qwen3moe.expert_used_count": 0}), be.Malformed, "experts used"),
        (dict(meta_extra={"qwen3moe.expert_used_count": 1000}), be.Malformed, "experts used"),
        (dict(drop_tensors=["token_embd.weight"]), be.Malformed, "token_embd.weight is absent"),
    ]
    for i, (kw, exc, needle) in enumerate(cases):
        _, path = tiny_file(gg, synth, tmp_path, f"bad{i}.gguf", **kw)
        with gg.Gguf.open(path) as g, pytest.raises(exc) as e:
            g.hparams()
        assert needle in str(e.value), (kw, str(e.value))


def test_a_dense_qwen3_file_reads_no_expert_keys(gg, synth, tmp_path):
    hp = dict(synth.TINY)
    meta = {k.replace("qwen3moe", "qwen3"): v for k, v in gg.synthetic_metadata(hp).items() if "expert" not in k}
    meta["general.architecture"] = "qwen3"
    path = tmp_path / "dense.gguf"
    gg.write_gguf(path, meta, [("token_embd.weight", [hp["n_embd"], 4], gg.GGML_F32, np.zeros(4 * hp["n_embd"], np.float32))])
    with gg.Gguf.open(path) as g:
        got = g.hparams()
        assert (got["arch"], got["n_expert"], got["n_expert_used"], got["n_ff_expert"], got["n_vocab"]) == ("qwen3", 0, 0, 0, 4)
        with pytest.raises(Exception, match="tensors missing, first"):
            g.verify_present()  # dense layers want ffn_gate / ffn_up / ffn_down


def test_verify_present_names_the_first_missing_tensors(gg, be, synth, tmp_path):
    drop = ["blk.0.attn_q.weight", "blk.1.ffn_down_exps.weight", "output_norm.weight", "blk.1.ffn_norm.weight"]
    _, path = tiny_file(gg, synth, tmp_path, "missing.gguf", drop_tensors=drop)
    with gg.Gguf.open(path) as g, pytest.raises(be.Malformed) as e:
        g.verify_present()
    msg = str(e.value)
    assert "4 tensors missing" in msg and '"output_norm.weight", "blk.0.attn_q.weight", "blk.1.ffn_norm.weight"' in msg
    # the optional per-head norms and output.weight may be absent
    _, path = tiny_file(gg, synth, tmp_path, "optional.gguf", drop_tensors=["output.weight", "blk.0.attn_q_norm.weight", "blk.1.attn_k_norm.weight"])
    with gg.Gguf.open(path) as g:
        g.verify_present()


def test_loading_without_a_device_is_refused_not_emulated(gg, be, synth, tmp_path):
    if be.available():
        pytest.skip("a device is present")
    _, path = tiny_file(gg, synth, tmp_path)
    from llamd_rs_b200.model import CudaModel

    with pytest.raises(be.Unsupported, match="no device"):
        CudaModel.open_gguf(path, 16)
    with pytest.raises(be.Malformed, match="max_kv of 0"):
        CudaModel.open_gguf(path, 0)
