"""CPU rehearsal of the expert-parallel exchange (gloo, any world size).

Each rank plays one GPU of `csrc/ep.cu`: it routes its own token with the
oracle, all-gathers (expert ids, Q8_K activation), computes the requested
experts it owns with the oracle's quantized matvec, returns the rows with an
all-to-all of fixed [n_used][n_embd] blocks, picks each slot's row from the
expert's owner and adds them in routing order. The result must equal the
oracle's single-process moe_ffn bit for bit.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist

    import oracle
    from llamd_rs_b200 import synth

    dist.init_process_group(backend="gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    hp = synth.TINY
    w = synth.make_model(hp, 21)
    om = oracle.Model(hp, w)
    om.kv_new(4)
    E, ffe, nu, ne = hp["n_embd"], hp["n_ff_expert"], hp["n_expert_used"], hp["n_expert"]
    per_rank = ne // world
    lo, hi = rank * per_rank, (rank + 1) * per_rank
    per = ffe * E // 256 * 210
    tok = 7 + 13 * rank
    x = oracle.dequantize(oracle.Q6K, w["tok_embd"][tok * (E // 256) * 210:], E)
    ok = True
    for il in range(hp["n_layer"]):
        x_next, tr = om.forward_layer(il, x, 0)          # the reference result for this rank's token
        ids, wts, xin = tr["experts"].astype(np.int32), tr["weights"], tr["ffn_norm"]
        qs, d, _ = oracle.quantize_q8k(xin)
        # dispatch: all-gather of ids and the Q8_K activation
        ids_all = [torch.zeros(nu, dtype=torch.int32) for _ in range(world)]
        qs_all = [torch.zeros(E, dtype=torch.int8) for _ in range(world)]
        d_all = [torch.zeros(E // 256, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(ids_all, torch.from_numpy(ids.copy()))
        dist.all_gather(qs_all, torch.from_numpy(qs.copy()))
        dist.all_gather(d_all, torch.from_numpy(d.copy()))
        # compute: the slots whose expert this rank owns, for every token
        lay = w["layers"][il]
        send = [torch.zeros(nu, E, dtype=torch.float32) for _ in range(world)]
        for t in range(world):
            for s in range(nu):
                e = int(ids_all[t][s])
                if not lo <= e < hi:
                    continue
                g = oracle.matvec_q6k_q8k(lay["ffn_gate_exps"][e * per:(e + 1) * per], qs_all[t].numpy(), d_all[t].numpy(), E, ffe)
                u = oracle.matvec_q6k_q8k(lay["ffn_up_exps"][e * per:(e + 1) * per], qs_all[t].numpy(), d_all[t].numpy(), E, ffe)
                act = oracle.mul(oracle.silu(g), u)
                send[t][s] = torch.from_numpy(oracle.matvec_q6k(lay["ffn_down_exps"][e * per:(e + 1) * per], act, ffe, E))
        # combine: fixed-size all-to-all, then pick by owner and add in routing order
        recv = [torch.zeros(nu, E, dtype=torch.float32) for _ in range(world)]
        dist.all_to_all(recv, send) if dist.get_backend() != "gloo" else _gloo_all_to_all(dist, recv, send, rank, world)
        acc = np.zeros(E, np.float32)
        for s in range(nu):
            row = recv[int(ids[s]) // per_rank][s].numpy()
            acc = (acc + (wts[s] * row).astype(np.float32)).astype(np.float32)
        ok &= np.array_equal(acc.view(np.uint32), tr["ffn_out"].view(np.uint32))
        ok &= np.array_equal((tr["ffn_inp"] + acc).astype(np.float32).view(np.uint32), x_next.view(np.uint32))
        x = x_next
    out = [None] * world
    dist.all_gather_object(out, bool(ok))
    if rank == 0:
        print("EP_PROTOCOL " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if all(out) else 1)


def _gloo_all_to_all(dist, recv, send, rank, world):
    # gloo has no all_to_all: the same exchange as pairwise send/recv
    import torch

    reqs = []
    for peer in range(world):
        if peer == rank:
            recv[peer].copy_(send[peer])
            continue
        reqs.append(dist.isend(send[peer].contiguous(), peer))
        reqs.append(dist.irecv(recv[peer], peer))
    for r in reqs:
        r.wait()


if __name__ == "__main__":
    main()
