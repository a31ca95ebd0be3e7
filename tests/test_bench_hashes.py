"""The hashes bench.py prints, pinned without a GPU.

bench.py's decode line carries `detail.inputs_hash` (crc32 of the prompt ids and of layer 0's attn_q bytes) and
`detail.tokens_hash` (crc32 of the token ids it decoded after the prompt). Both are functions of the seeded generator
and of the CPU path's greedy run over the same inputs, which is committed as tests/golden/decode_seed0.npz: a bench run
whose hashes differ from these ran other inputs or chose other tokens than llamd-cpu's arithmetic does."""
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "decode_seed0.npz")

INPUTS_HASH = "e64f1047"           # 512 prompt ids (seed 0, rank 0) + layer-0 attn_q of the 48-layer benchmark model
TOKENS_HASH_DEFAULT_RUN = "44b445f9"  # `python bench.py` (64 steps, 4 warm-up): 1 + 4 + 64 + 64 = 133 tokens after the prompt


def test_the_benchmark_inputs_are_the_pinned_ones():
    from llamd_rs_b200 import synth

    hp = dict(synth.QWEN3MOE_30B)
    prompt = synth.token_ids(512, hp["n_vocab"], 0, "prompt", 0)
    got = synth.checksum(np.asarray(prompt, np.int32), synth.layer_weights(hp, 0, 0, with_experts=False)["attn_q"])
    assert got == INPUTS_HASH
    g = np.load(GOLDEN)
    assert np.array_equal(g["prompt"], prompt), "the golden CPU run was made from the benchmark's own prompt"


def test_the_default_run_decodes_the_cpu_paths_tokens():
    """What bench.py hashes is the token chosen after the prompt, its warm-up tokens, the tokens of its end-to-end leg and
    of its device loop: consecutive greedy tokens. For the default run that is 133 of them; their hash, computed here from
    the CPU run, is the one a correct GPU run prints (bench.py also compares the tokens one by one)."""
    from llamd_rs_b200 import synth

    g = np.load(GOLDEN)
    chosen = g["chosen"]
    assert chosen.shape[0] >= 512 + 133
    decoded = np.asarray(chosen[511:511 + 133], np.int32)
    assert synth.checksum(decoded) == TOKENS_HASH_DEFAULT_RUN
    assert decoded[:3].tolist() == [143512, 91415, 122400]
