"""Host-side logic that needs no GPU: the synthetic generators, the oracle's
decode loop properties on the tiny model, byte accounting, and the two-rank
launch contract of bench.py's host plumbing (gloo, world size 2)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_generators_are_deterministic_and_in_range():
    from llamd_rs_b200 import synth

    a = synth.q6k_blocks(100, 0, "x", 1)
    assert np.array_equal(a, synth.q6k_blocks(100, 0, "x", 1)) and not np.array_equal(a, synth.q6k_blocks(100, 1, "x", 1))
    b = a.reshape(100, 210)
    sc = b[:, 192:208].view(np.int8)
    assert sc.min() >= -32 and sc.max() <= 31
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32)
    assert np.all(d >= 0) and np.all(np.isfinite(d)) and 1e-4 < d.mean() < 3e-3
    q = synth.q8_0_blocks(50, 0, "y").reshape(50, 34)
    assert q[:, 2:].view(np.int8).min() >= -127
    assert synth.token_ids(512, 151936, 0, "p").max() < 151936
    hp = synth.TINY
    full = synth.make_model(hp, 3)
    per = hp["n_ff_expert"] * hp["n_embd"] // 256 * 210
    e = synth.expert_blocks(hp, 3, 1, 2, 5)
    assert np.array_equal(full["layers"][1]["ffn_down_exps"][5 * per:6 * per], e), "an expert regenerates on its own"


def test_byte_accounting_matches_the_model():
    sys.path.insert(0, ROOT)
    import bench
    from llamd_rs_b200 import synth

    w, io = bench.matvec_bytes_per_token(synth.QWEN3MOE_30B)
    assert w == 48 * (15482880 + 30965760) + 255252480  # attention + 8 experts x 3, per layer; lm_head
    assert 0 < io < 0.01 * w


def test_oracle_decode_is_reproducible_and_expert_fn_equals_resident(orc):
    from llamd_rs_b200 import synth

    hp = synth.TINY
    w = synth.make_model(hp, 7)
    m1 = orc.Model(hp, w, threads=1)
    m1.kv_new(8)
    w2 = synth.make_model(hp, 7, with_experts=False)
    m2 = orc.Model(hp, w2, threads=3, expert_fn=lambda il, which, e: synth.expert_blocks(hp, 7, il, which, e))
    m2.kv_new(8)
    for pos, tok in enumerate([5, 99, 300]):
        a, b = m1.forward(tok, pos), m2.forward(tok, pos)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), "threads and lazy experts change nothing"
    with pytest.raises(ValueError):
        m1.forward(hp["n_vocab"], 3)
    with pytest.raises(ValueError):
        m1.forward(1, 8)  # beyond the cache


def test_moe_ffn_is_the_weighted_sum_in_routing_order(orc):
    from llamd_rs_b200 import synth

    hp = synth.TINY
    w = synth.make_model(hp, 9)
    m = orc.Model(hp, w)
    x = synth.normal_f32(hp["n_embd"], 9, "x")
    experts, weights = [3, 6], np.array([0.7, 0.3], np.float32)
    got = m.moe_ffn(0, x, experts, weights)
    per = hp["n_ff_expert"] * hp["n_embd"] // 256 * 210
    acc = np.zeros(hp["n_embd"], np.float32)
    for e, wt in zip(experts, weights):
        lay = w["layers"][0]
        g = orc.matvec_q6k(lay["ffn_gate_exps"][e * per:(e + 1) * per], x, hp["n_embd"], hp["n_ff_expert"])
        u = orc.matvec_q6k(lay["ffn_up_exps"][e * per:(e + 1) * per], x, hp["n_embd"], hp["n_ff_expert"])
        dn = orc.matvec_q6k(lay["ffn_down_exps"][e * per:(e + 1) * per], orc.mul(orc.silu(g), u), hp["n_ff_expert"], hp["n_embd"])
        acc = (acc + (wt * dn).astype(np.float32)).astype(np.float32)
    assert np.array_equal(got.view(np.uint32), acc.view(np.uint32))
    with pytest.raises(ValueError):
        m.moe_ffn(0, x, [hp["n_expert"]], [1.0])


_RANK_SCRIPT = r"""
import os, sys, json
import torch, torch.distributed as dist
dist.init_process_group(backend="gloo")
rank, world = dist.get_rank(), dist.get_world_size()
# the bench's host plumbing: barrier, MAX of per-rank time, sum of per-rank work
t = torch.tensor([1.0 + rank], dtype=torch.float64)
dist.barrier()
dist.all_reduce(t, op=dist.ReduceOp.MAX)
if rank == 0:
    print(json.dumps({"max_s": float(t.item()), "world": world}))
dist.barrier()
dist.destroy_process_group()
"""


def test_two_rank_contract_on_gloo(tmp_path):
    """world_size 2 on CPU: max-over-ranks timing and rank-0-only output."""
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                          "127.0.0.1", "--master-port", "29741", str(script)], capture_output=True, text=True, env=env, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1 and json.loads(lines[0]) == {"max_s": 2.0, "world": 2}


def test_reference_arm_other_ranks_exit_quietly():
    """Under torchrun only rank 0 runs the CPU reference arm."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                         capture_output=True, text=True, env=env, timeout=120)
    assert out.returncode == 0 and out.stdout.strip() == ""


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_protocol_on_gloo(world):
    """The dispatch / owned-expert compute / ordered combine of the expert-parallel path, rehearsed with the
    oracle over gloo: every rank's MoE output equals the single-process oracle bit for bit."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
                          "127.0.0.1", "--master-port", str(29760 + world), os.path.join(ROOT, "tests", "ep_protocol_worker.py")],
                         capture_output=True, text=True, env=env, timeout=300)
    lines = [l for l in out.stdout.splitlines() if l.startswith("EP_PROTOCOL ")]
    assert out.returncode == 0 and lines, (out.stdout[-1000:], out.stderr[-2000:])
    assert json.loads(lines[0][len("EP_PROTOCOL "):]) == [True] * world


# ---- the peer-memory exchange of expert parallelism, as a model -------------------------------
# csrc/ep.cu + the waits in matvec_q6k.cu / quantize.cu order their accesses with two counters per rank and no
# barrier. This is that protocol with the GPU taken out: ranks are step lists, a random scheduler picks any step whose
# wait condition holds, and every read checks that it sees the layer it belongs to (a record or a row replaced too
# early, or read before it arrived, shows up as a wrong tag).
def _simulate_peer_exchange(world, layers, ctas, seed, mode="per_rank"):
    import random

    rng = random.Random(seed)
    n_used = 2
    disp = [0] * world          # dispatch counter of each rank (only grows)
    epoch = [0] * world         # each rank's own epoch (bumped by its push)
    arrive = [0] * world        # arrival counter of each home rank (cleared by its norm)
    rec = [[-1] * world for _ in range(world)]             # rec[dst][src]: layer tag of src's request record at dst
    out = [[-1] * n_used for _ in range(world)]            # out[home][slot]: layer tag of the expert rows
    owner = lambda home, slot, layer: (home + slot + layer) % world  # which rank owns that slot's expert
    # per_cta (the kernels' default): every CTA arrives on its slot's home; per_rank (option ep_rank_arrive): a rank counts its
    # own down CTAs and arrives once on every home when the last is done; owners_only: only the CTAs that store rows do (the
    # broken variant)
    target_rows = {"per_rank": world, "per_cta": world * n_used * ctas, "owners_only": n_used * ctas}[mode]
    local_done = [0] * world

    def steps(r):
        for l in range(layers):
            yield ("push", l)
            # gate/up: one step per (home) after the dispatch wait; reads the home's record
            for home in range(world):
                yield ("gate_up", l, home)
            # down: one step per (home, slot, cta): reads the id, owners store rows, then arrive
            order = [(h, s, c) for h in range(world) for s in range(n_used) for c in range(ctas)]
            rng.shuffle(order)
            for h, s, c in order:
                yield ("down", l, h, s, c)
            yield ("norm", l)

    its = [steps(r) for r in range(world)]
    cur = [next(it) for it in its]
    done = [False] * world
    executed = 0
    while not all(done):
        ready = []
        for r in range(world):
            if done[r]:
                continue
            st = cur[r]
            if st[0] == "gate_up" and disp[r] < epoch[r] * world:
                continue  # the dispatch wait
            if st[0] == "norm" and arrive[r] < target_rows:
                continue  # the combine wait
            ready.append(r)
        assert ready, "deadlock: every rank waits"
        r = rng.choice(ready)
        st = cur[r]
        if st[0] == "push":
            for dst in range(world):
                rec[dst][r] = st[1]
                disp[dst] += 1
            epoch[r] += 1
        elif st[0] == "gate_up":
            assert rec[r][st[2]] == st[1], f"rank {r} layer {st[1]}: record of rank {st[2]} is from layer {rec[r][st[2]]}"
        elif st[0] == "down":
            _, l, h, s, c = st
            assert rec[r][h] == l, f"rank {r} layer {l}: a down CTA read a record of layer {rec[r][h]}"
            if owner(h, s, l) == r:
                out[h][s] = l
            if mode == "per_rank":
                local_done[r] += 1
                if local_done[r] == world * n_used * ctas:  # the CTA that completes the count signals every home
                    local_done[r] = 0
                    for hh in range(world):
                        arrive[hh] += 1
            elif owner(h, s, l) == r or mode == "per_cta":
                arrive[h] += 1
        else:  # norm: all rows of this layer are in; clear the counter
            assert all(t == st[1] for t in out[r]), f"rank {r} layer {st[1]}: rows {out[r]}"
            arrive[r] = 0
        executed += 1
        try:
            cur[r] = next(its[r])
        except StopIteration:
            done[r] = True
    return executed


@pytest.mark.parametrize("world,ctas", [(2, 1), (2, 3), (4, 2), (8, 1)])
def test_peer_exchange_protocol_orders_reads_and_writes(world, ctas):
    for seed in range(40):
        _simulate_peer_exchange(world, layers=5, ctas=ctas, seed=seed)
        _simulate_peer_exchange(world, layers=5, ctas=ctas, seed=seed, mode="per_cta")


def test_peer_exchange_needs_every_cta_to_arrive():
    """If only the owners' CTAs counted, a rank could replace its record while a late CTA of another rank has not
    read the old one: the model finds such a schedule."""
    with pytest.raises(AssertionError):
        for seed in range(400):
            _simulate_peer_exchange(4, layers=6, ctas=2, seed=seed, mode="owners_only")


def test_every_model_option_is_documented():
    """Every name llamd_model_set_option accepts is described in include/llamd_cuda_model.h and named in INTEGRATION.md."""
    import os
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = open(os.path.join(root, "llamd_rs_b200", "csrc", "model.cu")).read()
    names = sorted(set(re.findall(r'!strcmp\(name, "([a-z0-9_]+)"\)', src)))
    assert len(names) >= 20
    hdr = open(os.path.join(root, "include", "llamd_cuda_model.h")).read()
    integ = open(os.path.join(root, "INTEGRATION.md")).read()
    missing_h = [n for n in names if f'"{n}"' not in hdr]
    missing_i = [n for n in names if f"`{n}`" not in integ]
    assert not missing_h, f"options not described in the header: {missing_h}"
    assert not missing_i, f"options not named in INTEGRATION.md: {missing_i}"
