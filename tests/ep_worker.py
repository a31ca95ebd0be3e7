"""One rank of the expert-parallel parity check (launched by test_gpu_ep.py
under torchrun, one process per GPU).

Each rank first decodes ITS sequence on a full single-GPU model, then joins the
NCCL communicator, reloads the model with only its share of the experts and
decodes the same sequence again together with the other ranks. Tokens and
logits must be identical, bit for bit: the exchange moves Q8_K activations and
f32 rows without touching them, and the home rank adds the expert outputs in
routing order exactly as the single-GPU pass does. The same is then repeated
with both collectives replaced by stores into the other ranks' buffers over
NVLink (CUDA IPC) and arrival counters, and in that form the tiled prefill is
checked too: every rank's tile gathered on every rank, the owned experts run on
the grouped GEMM over all ranks' tokens, rows stored to the token's home rank.
Batches of sequences (forward_batch, 3 and 12 per rank, each rank its own) go
through the same tile exchange: one rendezvous each way per layer for all of a
rank's sequences.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch.distributed as dist

    from llamd_rs_b200 import backend, synth
    from llamd_rs_b200 import model as M

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    full_size = len(sys.argv) > 1 and sys.argv[1] == "full"
    dist.init_process_group(backend="gloo")
    backend.set_device(local)
    backend.stream_init()
    hp = dict(synth.QWEN3MOE_30B, n_layer=3) if full_size else synth.TINY
    n_prompt, n_gen = 5, 6
    prompt = synth.token_ids(n_prompt, hp["n_vocab"], 11, "ep", rank).tolist()
    # prefill: ranks bring prompts of different lengths that cut into the same number of tiles
    max_kv, pf_tile = (160, 64) if full_size else (32, 4)
    n_pf = (100 if full_size else 7) + rank % 2
    pf_prompt = synth.token_ids(n_pf, hp["n_vocab"], 12, "ep.prefill", rank).tolist()

    def prefill_then_two(m):
        tok = m.prefill(pf_prompt, 0)
        logits = m.logits()[0].copy()
        t1 = m.forward(tok, n_pf)
        return [tok, t1, m.forward(t1, n_pf + 1)], logits

    def decode(m):
        toks, tok = [], None
        for pos in range(n_prompt + n_gen):
            tok = m.forward(prompt[pos] if pos < n_prompt else tok, pos)
            toks.append(tok)
        return toks, m.logits()[0].copy()

    n_batch = 12
    batch_tokens = synth.token_ids(n_batch * 4, hp["n_vocab"], 13, "ep.batch", rank).reshape(4, n_batch)

    def batches(m):
        """Four steps of 12 sequences, then the first 3 sequences one step further: tokens and logits of every step."""
        out = []
        for pos in range(4):
            toks = m.forward_batch(batch_tokens[pos].tolist(), [pos] * n_batch)
            out.append((toks.tolist(), m.logits(n_batch).copy()))
        toks = m.forward_batch(batch_tokens[0][:3].tolist(), [4] * 3)
        out.append((toks.tolist(), m.logits(3).copy()))
        return out

    m = M.CudaModel.load_synthetic(hp, 5, max_kv=max_kv, max_seq=n_batch)
    want_batches = batches(m)
    want_toks, want_logits = decode(m)
    single_bytes = m.weight_bytes()
    m.use_graph = False
    assert decode(m)[0] == want_toks
    m.use_graph = True
    want_pf, want_pf_logits = prefill_then_two(m)
    m.free()

    def share(b):
        obj = [b]
        dist.broadcast_object_list(obj, src=0)
        return obj[0]

    M.ep_init(rank, world, share)
    m = M.CudaModel.load_synthetic(hp, 5, max_kv=max_kv, max_seq=n_batch)
    full_bytes = hp["n_layer"] * 3 * hp["n_expert"] * (hp["n_ff_expert"] * hp["n_embd"] // 256 * 210)
    got_toks, got_logits = decode(m)            # captured graph with the NCCL exchange inside
    m.use_graph = False
    plain_toks, plain_logits = decode(m)        # plain queueing

    # the same with both collectives replaced by peer stores + arrival counters
    def gather(b):
        out = [None] * world
        dist.all_gather_object(out, b)
        return out

    m.ep_p2p_attach(gather)
    dist.barrier()
    m.use_graph = True
    p2p_toks, p2p_logits = decode(m)
    m.use_graph = False
    p2p_plain_toks, _ = decode(m)
    # tiled prefill over peer memory: one tile of the whole capacity, then tiles of pf_tile tokens
    m.use_graph = True
    pf_results = []
    for tile in (m.ep_tile_cap(), pf_tile):
        m.prefill_tile = tile
        pf_results.append(prefill_then_two(m))
    pf_ok = all(t == want_pf and np.array_equal(lg.view(np.uint32), want_pf_logits.view(np.uint32)) for t, lg in pf_results)
    got_batches = batches(m)
    batch_ok = all(gt == wt and np.array_equal(gl.view(np.uint32), wl.view(np.uint32)) for (gt, gl), (wt, wl) in zip(got_batches, want_batches))
    pf_ok = pf_ok and batch_ok
    ok = (pf_ok and got_toks == want_toks and plain_toks == want_toks and p2p_toks == want_toks and p2p_plain_toks == want_toks
          and np.array_equal(got_logits.view(np.uint32), want_logits.view(np.uint32))
          and np.array_equal(plain_logits.view(np.uint32), want_logits.view(np.uint32))
          and np.array_equal(p2p_logits.view(np.uint32), want_logits.view(np.uint32)))
    res = dict(rank=rank, ok=bool(ok), prefill_ok=bool(pf_ok), batch_ok=bool(batch_ok), prefill_tokens=[t for t, _ in pf_results], prefill_want=want_pf,
               tile_cap=m.ep_tile_cap(), tokens=got_toks, p2p_tokens=p2p_toks, want=want_toks, weight_bytes=m.weight_bytes(), single_bytes=single_bytes,
               full_expert_bytes=full_bytes)
    m.free()
    M.ep_finalize()
    out = [None] * world
    dist.all_gather_object(out, res)
    if rank == 0:
        print("EP_RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if all(r["ok"] for r in out) else 1)


if __name__ == "__main__":
    main()
