"""Generate tests/golden/decode_seed0.npz: the CPU oracle's greedy run of the decode benchmark.

The 48-layer, 128-expert random-init model (seed 0) reads the benchmark's 512 prompt ids and then decodes 256
greedy tokens, all on the CPU oracle (oracle/llamd_oracle.c, the restatement of the reference's scalar path).
Recorded: the prompt, the token chosen after every position from the last prompt position on, the routed expert
ids of every layer at every position, and the top-1 / top-2 logit margin at every decoded position.

Needs ~26 GB of host memory (every expert is held) and about 15 minutes on 8 cores:

    python tests/golden/make_decode_golden.py [--threads N] [--decode 256]
"""
import argparse
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main():
    import oracle
    from llamd_rs_b200 import synth

    ap = argparse.ArgumentParser()
    ap.add_argument("--threads", type=int, default=os.cpu_count() or 1)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--decode", type=int, default=256)
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden", "decode_seed0.npz"))
    args = ap.parse_args()
    hp, seed = dict(synth.QWEN3MOE_30B), 0
    t0 = time.time()
    w = synth.make_model(hp, seed, with_experts=True)
    print(f"weights generated in {time.time() - t0:.0f}s", flush=True)
    om = oracle.Model(hp, w, threads=args.threads)
    n_pos = args.prompt + args.decode
    om.kv_new(n_pos)
    prompt = synth.token_ids(args.prompt, hp["n_vocab"], seed, "prompt", 0)
    E, L, nu = hp["n_embd"], hp["n_layer"], hp["n_expert_used"]
    row = (E // 256) * 210
    experts = np.zeros((n_pos, L, nu), np.uint8)
    chosen = np.full(n_pos, -1, np.int64)   # chosen[p] = greedy token after position p (from the last prompt position on)
    margin = np.zeros(n_pos, np.float32)
    tok = None
    for pos in range(n_pos):
        t = int(prompt[pos]) if pos < args.prompt else tok
        x = oracle.dequantize(oracle.Q6K, w["tok_embd"][t * row:(t + 1) * row], E)
        for il in range(L):
            x, tr = om.forward_layer(il, x, pos)
            experts[pos, il] = tr["experts"]
        if pos >= args.prompt - 1:
            normed = oracle.mul(oracle.rms_norm(x, hp["rms_eps"]), w["output_norm"])
            logits = oracle.matvec_q6k(w["output"], normed, E, hp["n_vocab"], threads=args.threads)
            tok = oracle.argmax(logits)
            chosen[pos] = tok
            top2 = np.partition(logits, -2)[-2:]
            margin[pos] = top2[1] - top2[0]
        if pos % 32 == 31 or pos == n_pos - 1:
            print(f"position {pos + 1}/{n_pos} after {time.time() - t0:.0f}s", flush=True)
            np.savez_compressed(args.out, prompt=prompt.astype(np.int32), chosen=chosen.astype(np.int32), experts=experts,
                                margin=margin, done=np.int32(pos + 1), seed=np.int32(seed))


if __name__ == "__main__":
    main()
