"""Expert parallelism on real GPUs: 2 (and 4 if present) ranks, one process per
GPU, NCCL exchange per MoE layer. Each rank's tokens and logits must equal the
single-GPU model's, bit for bit (see ep_worker.py). Needs at least two GPUs."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_ranks(n, mode, port):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "ep_worker.py"), mode]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=900)
    line = [l for l in out.stdout.splitlines() if l.startswith("EP_RESULT ")]
    assert out.returncode == 0 and line, (out.stdout[-1500:], out.stderr[-3000:])
    return json.loads(line[0][len("EP_RESULT "):])


@pytest.mark.parametrize("n,mode", [(2, "tiny"), (2, "full"), (4, "tiny")])
def test_expert_parallel_decode_equals_single_gpu(n, mode):
    from llamd_rs_b200 import backend

    have = backend.device_count()
    if have == 0:
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    if have < n:
        pytest.skip(f"expert parallelism over {n} ranks needs {n} GPUs, this box has {have}")
    res = run_ranks(n, mode, 29750 + n)
    assert len(res) == n
    for r in res:
        assert r["ok"], r
        assert r["tokens"] == r["want"]
    # each rank keeps exactly 1/n of the expert bytes and every other weight
    assert all(r["weight_bytes"] == r["single_bytes"] - r["full_expert_bytes"] * (n - 1) // n for r in res)
