"""GPU parity of the resident decode model against the oracle's decode loop.

A small Qwen3MoE-shaped model (2 layers, 8 experts, 2 active) is decoded token
by token on both sides from the same seeded weights. Expert ids and greedy
token ids must be identical; hidden states, K/V and logits are compared bit
for bit where no exp() is upstream, and at the reference's named tolerances
(crates/llamd-core/src/tolerance.rs) after one.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LAYER = 1e-4      # tolerance.rs:100
LOGITS = 2e-3     # tolerance.rs:109
ATTENTION = 1e-5  # tolerance.rs:97


def max_dev(a, b):
    """llamd_core::tolerance::max_deviation (tolerance.rs:135-151)."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.maximum(np.abs(a), np.abs(b)), 1.0)))


@pytest.fixture(scope="module")
def tiny():
    from llamd_rs_b200 import backend, synth
    from llamd_rs_b200.model import CudaModel
    import oracle

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    hp = synth.TINY
    w = synth.make_model(hp, seed=7)
    gm = CudaModel.load_batched(hp, w, max_kv=64, max_seq=4)
    om = oracle.Model(hp, w, threads=4)
    yield hp, w, gm, om
    gm.free()


def test_bad_arguments_are_refused(tiny):
    from llamd_rs_b200 import backend
    from llamd_rs_b200.model import CudaModel

    hp, w, gm, om = tiny
    with pytest.raises(backend.Malformed):
        CudaModel(hp, 0)
    with pytest.raises(backend.Malformed):
        CudaModel(hp, 16, backend.MAX_BATCH + 1)
    with pytest.raises(backend.Malformed):
        gm.forward(1, 64)
    with pytest.raises(backend.Other):
        gm.forward(hp["n_vocab"], 0)
    assert gm.weight_bytes() > 0 and gm.hparams()["n_layer"] == 2


def test_first_token_layer_by_layer(tiny):
    """Position 0: softmax over one key is exactly 1, so nothing upstream of the
    router depends on exp(); the routing itself does."""
    hp, w, gm, om = tiny
    om.kv_new(64)
    gm.set_trace(True)
    tok = 17
    got_tok = gm.forward(tok, 0)
    gx, gids = gm.read_trace()
    gm.set_trace(False)
    import oracle

    x = oracle.dequantize(oracle.Q6K, w["tok_embd"][tok * hp["n_embd"] // 256 * 210:], hp["n_embd"])
    for il in range(hp["n_layer"]):
        x, tr = om.forward_layer(il, x, 0)
        assert gids[il, 0].tolist() == tr["experts"].tolist(), f"layer {il} expert ids"
        assert max_dev(gx[il, 0], x) <= LAYER, f"layer {il} hidden state"
        gk, gv = gm.read_kv(il, 1)
        ok, ov = om.kv_layer(il, 1)
        assert np.array_equal(gv.view(np.uint32), ov.view(np.uint32)) or il > 0, "layer 0 V is exp-free: bit-exact"
        assert max_dev(gk, ok) <= ATTENTION and max_dev(gv, ov) <= ATTENTION
    om.kv_new(64)
    logits = om.forward(tok, 0)
    assert max_dev(gm.logits()[0], logits) <= LOGITS
    assert got_tok == oracle.argmax(logits)


def test_greedy_decode_matches_token_for_token(tiny):
    """Prompt of 6 ids, then 10 greedy tokens: ids EXACT, logits at LOGITS."""
    import oracle
    from llamd_rs_b200 import synth

    hp, w, gm, om = tiny
    prompt = synth.token_ids(6, hp["n_vocab"], 3, "prompt").tolist()
    om.kv_new(64)
    want, got = [], []
    worst = 0.0
    tok_o = tok_g = None
    for pos in range(16):
        t_in_o = prompt[pos] if pos < len(prompt) else tok_o
        t_in_g = prompt[pos] if pos < len(prompt) else tok_g
        lo = om.forward(t_in_o, pos)
        tok_o = oracle.argmax(lo)
        tok_g = gm.forward(t_in_g, pos)
        worst = max(worst, max_dev(gm.logits()[0], lo))
        want.append(tok_o)
        got.append(tok_g)
        assert tok_g == tok_o, f"token {pos}: gpu {got} cpu {want}"
    assert worst <= LOGITS, f"logits deviate by {worst}"


def test_graph_replay_equals_plain_queueing(tiny):
    hp, w, gm, om = tiny
    gm.use_graph = False
    a = [gm.forward(5 + p, p) for p in range(5)]
    la = gm.logits()[0]
    gm.use_graph = True
    b = [gm.forward(5 + p, p) for p in range(5)]
    lb = gm.logits()[0]
    assert a == b and np.array_equal(la.view(np.uint32), lb.view(np.uint32))


def test_batch_equals_single(tiny):
    """crates/llamd-testing/tests/batch_decode.rs:102-125: N sequences in one
    pass give the tokens (and here the logits, bit for bit) of N single passes."""
    hp, w, gm, om = tiny
    seqs = [[3, 9, 27], [100, 200, 300], [7, 7, 7], [511, 0, 255]]
    single_tokens, single_logits = [], []
    for s in seqs:
        toks = []
        for pos, t in enumerate(s):
            toks.append(gm.forward(t, pos))
        single_tokens.append(toks)
        single_logits.append(gm.logits()[0].copy())
    # batched: all four sequences advance together (each in its own KV slot)
    for pos in range(3):
        out = gm.forward_batch([s[pos] for s in seqs], [pos] * 4)
        assert out.tolist() == [st[pos] for st in single_tokens]
    lb = gm.logits(4)
    for i in range(4):
        assert np.array_equal(lb[i].view(np.uint32), single_logits[i].view(np.uint32)), f"sequence {i} logits"


def test_fused_tails_change_nothing(tiny):
    """The decode pass with the attention-quantize and SiLU-quantize tails inside their producers (option
    fuse_tails) and with the separate launches (default): same tokens, same logits, bit for bit."""
    hp, w, gm, om = tiny
    runs = {}
    for fuse in (0, 1, 0):
        gm.set_option("fuse_tails", fuse)
        toks, tok = [], 3
        for pos in range(6):
            tok = gm.forward(tok, pos)
            toks.append(tok)
        runs.setdefault(fuse, []).append((toks, gm.logits()[0].copy()))
    gm.set_option("fuse_tails", 0)
    ref_t, ref_l = runs[1][0]
    for t, l in runs[0]:
        assert t == ref_t and np.array_equal(l.view(np.uint32), ref_l.view(np.uint32))


@pytest.mark.parametrize("option", ["fuse_norm_router", "fuse_rope_attn", "fuse_norm_qkv", "fuse_silu_down", "early_loads", "fuse_attn_quant", "sort_slots", "head_gemm", "dense_gemm"])
def test_fused_launches_change_nothing(tiny, option):
    """The decode pass with the FFN norm and the router as one launch (option fuse_norm_router), with QK-norm, RoPE and
    the KV store inside the attention-scores launch (option fuse_rope_attn), and with the attention norm and the MoE combine
    inside the QKV matvec (option fuse_norm_qkv; off by default), and with the loads that do not depend on the launch in
    front issued before the dependency wait (option early_loads), and with the expert launches taking their slots in expert
    order (option sort_slots), and with the output projection, or the attention projections, on the integer GEMM over folded
    copies of their matrices (options head_gemm, dense_gemm) -- against the separate launches, the late loads, the slots in routing order and the output matvec: same tokens, same hidden states after every layer, same routed experts, same logits and cache rows, bit for
    bit; one and four sequences. (Positions beyond a 64-position tile, where the token's own row moves from tile to tile, are
    covered by the 768-position run against the CPU fixture, which uses the defaults.)"""
    hp, w, gm, om = tiny
    runs = {}
    default = 0 if option in ("fuse_norm_qkv", "fuse_silu_down", "fuse_attn_quant") else 1  # (measured no faster, so off unless asked for)
    if option == "sort_slots":
        default = 8  # (the number of sequences from which the expert launches take their slots in expert order; 1: always)
    if option == "head_gemm":
        default = 4  # (the number of sequences from which the output projection runs on the integer GEMM; 1: always)
    if option == "dense_gemm":
        default = 8  # (the same for the attention projections)
    for fuse in (1, 0, 1):
        gm.set_option(option, fuse)
        gm.set_trace(True)
        toks, tok, traces = [], 3, []
        for pos in range(6):
            tok = gm.forward(tok, pos)
            toks.append(tok)
            x, ids = gm.read_trace()
            traces.append((x.copy(), ids.copy()))
        gm.set_trace(False)
        batch = [gm.forward_batch([5 + pos, 9, 100 + pos, 7], [pos] * 4).tolist() for pos in range(3)]
        kv = [gm.read_kv(il, 3) for il in range(hp["n_layer"])]
        runs.setdefault(fuse, []).append((toks, traces, gm.logits(4).copy(), batch, kv))
    gm.set_option(option, default)
    ref = runs[0][0]
    for toks, traces, logits, batch, kv in runs[1]:
        assert toks == ref[0] and batch == ref[3]
        assert np.array_equal(logits.view(np.uint32), ref[2].view(np.uint32))
        for (k, v), (rk, rv) in zip(kv, ref[4]):
            assert np.array_equal(k.view(np.uint32), rk.view(np.uint32)) and np.array_equal(v.view(np.uint32), rv.view(np.uint32))
        for (x, ids), (rx, rids) in zip(traces, ref[1]):
            assert np.array_equal(x.view(np.uint32), rx.view(np.uint32)) and np.array_equal(ids, rids)


@pytest.mark.parametrize("kv_f16", [0, 1])
def test_attention_output_leaves_its_launch_quantized(kv_f16):
    """Heads of 128: the eight CTAs that make a 256-element block of the attention output form a cluster, exchange their
    largest magnitudes through distributed shared memory and write the block's Q8_K form themselves (option fuse_attn_quant;
    off by default, measured slower) -- against the separate quantize launch: the same tokens, hidden states, experts, logits and cache rows, bit
    for bit; one and four sequences; against the oracle for the first tokens. Also with the loads before the wait off."""
    import oracle
    from llamd_rs_b200 import synth
    from llamd_rs_b200.model import CudaModel

    hp = dict(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, head_dim=128, n_expert=8, n_expert_used=2, n_ff_expert=256, n_vocab=512,
              rope_freq_base=1e7, rms_eps=1e-6)
    w = synth.make_model(hp, seed=11)
    gm = CudaModel.load_batched(hp, w, max_kv=96, max_seq=4)
    try:
        if kv_f16:
            gm.set_option("kv_f16", 1)
        runs = []
        for fuse, early in ((1, 1), (0, 1), (1, 0), (1, 1)):
            gm.set_option("fuse_attn_quant", fuse)
            gm.set_option("early_loads", early)
            gm.set_trace(True)
            toks, tok, traces = [], 3, []
            for pos in range(70):  # (past one 64-position tile of the scores launch)
                tok = gm.forward(tok, pos)
                toks.append(tok)
                if pos < 6 or pos > 62:
                    x, ids = gm.read_trace()
                    traces.append((x.copy(), ids.copy()))
            gm.set_trace(False)
            batch = [gm.forward_batch([5 + pos, 9, 100 + pos, 7], [pos] * 4).tolist() for pos in range(3)]
            runs.append((toks, traces, gm.logits(4).copy(), batch, [gm.read_kv(il, 3) for il in range(hp["n_layer"])]))
        ref = runs[1]
        for toks, traces, logits, batch, kv in (runs[0], runs[2], runs[3]):
            assert toks == ref[0] and batch == ref[3]
            assert np.array_equal(logits.view(np.uint32), ref[2].view(np.uint32))
            for (k, v), (rk, rv) in zip(kv, ref[4]):
                assert np.array_equal(k.view(np.uint32), rk.view(np.uint32)) and np.array_equal(v.view(np.uint32), rv.view(np.uint32))
            for (x, ids), (rx, rids) in zip(traces, ref[1]):
                assert np.array_equal(x.view(np.uint32), rx.view(np.uint32)) and np.array_equal(ids, rids)
        if not kv_f16:
            om = oracle.Model(hp, w, threads=4)
            om.kv_new(96)
            tok = 3
            for pos in range(8):
                tok = oracle.argmax(om.forward(tok, pos))
                assert tok == ref[0][pos], f"position {pos}"
    finally:
        gm.free()


@pytest.mark.parametrize("kv_f16", [0, 1])
def test_batch_attention_per_kv_head(kv_f16):
    """Eight query heads of 128 per kv head: a batch of sequences runs attention as one CTA per kv head for all of them
    (option attn_gqa, the default, from four sequences on). Sequences at different positions, across the 64-position score tiles and the
    256-position value tiles: each sequence's tokens, logits and cache rows equal a single-sequence run's, bit for bit, and
    the per-head kernels' on the same batch."""
    from llamd_rs_b200 import synth
    from llamd_rs_b200.model import CudaModel

    hp = dict(n_layer=2, n_embd=256, n_head=8, n_head_kv=1, head_dim=128, n_expert=8, n_expert_used=2, n_ff_expert=256, n_vocab=512,
              rope_freq_base=1e7, rms_eps=1e-6)
    w = synth.make_model(hp, seed=13)
    gm = CudaModel.load_batched(hp, w, max_kv=320, max_seq=4)
    try:
        if kv_f16:
            gm.set_option("kv_f16", 1)
        lens = [300, 70, 5, 130]  # the sequences end at different positions
        prompts = [synth.token_ids(n, hp["n_vocab"], 40 + i, "gqa").tolist() for i, n in enumerate(lens)]
        single = []
        for s_, pr in enumerate(prompts):
            for pos, t in enumerate(pr):
                tok = gm.forward(t, pos)
            single.append((tok, gm.logits()[0].copy(), [gm.read_kv(il, len(pr)) for il in range(hp["n_layer"])]))
        runs = {}
        for gqa in (1, 0):
            gm.set_option("attn_gqa", gqa)
            # the four sequences advance together while they last; a finished one repeats its last token at its last position
            for step in range(max(lens)):
                toks = [pr[min(step, len(pr) - 1)] for pr in prompts]
                poss = [min(step, len(pr) - 1) for pr in prompts]
                out = gm.forward_batch(toks, poss)
            runs[gqa] = (out.tolist(), gm.logits(4).copy())
        gm.set_option("attn_gqa", 1)
        assert runs[1][0] == runs[0][0] and np.array_equal(runs[1][1].view(np.uint32), runs[0][1].view(np.uint32))
        for s_ in range(4):  # (a finished sequence repeated its last position: the same row, the same logits)
            assert runs[1][0][s_] == single[s_][0], f"sequence {s_}"
            assert np.array_equal(runs[1][1][s_].view(np.uint32), single[s_][1].view(np.uint32)), f"sequence {s_}: logits"
            for il in range(hp["n_layer"]):
                k, v = gm.read_kv(il, lens[s_], s_)
                rk, rv = single[s_][2][il]
                assert np.array_equal(k.view(np.uint32), rk.view(np.uint32)) and np.array_equal(v.view(np.uint32), rv.view(np.uint32))
    finally:
        gm.free()


def test_prefill_equals_sequential_decode(tiny):
    """crates/llamd-testing/tests/vulkan_prefill.rs:48-136: prefill gives the token (and here the logits and the
    K/V cache, bit for bit) of sequential decode, for (tile, length) pairs that straddle tile and chunk boundaries."""
    from llamd_rs_b200 import backend, synth

    hp, w, gm, om = tiny
    prompt = synth.token_ids(37, hp["n_vocab"], 5, "prefill").tolist()
    seq_tok, seq_logits = {}, {}
    for pos, t in enumerate(prompt):
        seq_tok[pos + 1] = gm.forward(t, pos)
        seq_logits[pos + 1] = gm.logits()[0].copy()
    kv_ref = [gm.read_kv(il, len(prompt)) for il in range(hp["n_layer"])]
    for tile, length in [(1, 1), (1, 5), (2, 5), (4, 4), (4, 5), (8, 7), (8, 8), (8, 9), (8, 17), (16, 33), (16, 37), (64, 37), (512, 37)]:
        gm.prefill_tile = tile
        for gemm, attn in ((True, True), (False, True), (True, False)):  # integer tensor path / dp4a; tiled / per-token attention
            gm.set_prefill_gemm(gemm)
            gm.set_prefill_attn(attn)
            got = gm.prefill(prompt[:length], 0)
            assert got == seq_tok[length], f"tile {tile} length {length} gemm {gemm} attn {attn}"
            assert np.array_equal(gm.logits()[0].view(np.uint32), seq_logits[length].view(np.uint32)), f"tile {tile} length {length}: logits"
    gm.set_prefill_gemm(True)
    gm.set_prefill_attn(True)
    # the expert matrices folded once and kept (option prefill_prefold): the grouped GEMM copies operands instead of
    # folding them, the same bits
    gm.set_option("prefill_prefold", 1)
    for tile, length in [(4, 5), (8, 17), (16, 37), (512, 37)]:
        gm.prefill_tile = tile
        got = gm.prefill(prompt[:length], 0)
        assert got == seq_tok[length], f"prefold: tile {tile} length {length}"
        assert np.array_equal(gm.logits()[0].view(np.uint32), seq_logits[length].view(np.uint32)), f"prefold: tile {tile} length {length}: logits"
    gm.set_option("prefill_prefold", 0)
    gm.prefill_tile = 512
    assert gm.prefill(prompt, 0) == seq_tok[len(prompt)]
    for il in range(hp["n_layer"]):
        k, v = gm.read_kv(il, len(prompt))
        assert np.array_equal(k.view(np.uint32), kv_ref[il][0].view(np.uint32)) and np.array_equal(v.view(np.uint32), kv_ref[il][1].view(np.uint32))
    # chunked: a later call continues at base_pos, and decode continues after a prefill
    gm.prefill_tile = 8
    gm.prefill(prompt[:20], 0)
    assert gm.prefill(prompt[20:], 20) == seq_tok[37]
    gm.prefill(prompt[:12], 0)
    assert gm.forward(prompt[12], 12) == seq_tok[13]
    with pytest.raises(backend.Other):
        gm.prefill(prompt, 40)  # runs past the 64 allocated positions
    with pytest.raises(backend.Malformed):
        gm.prefill([], 0)
    gm.prefill_tile = 512
