"""Failure detection of the expert-parallel path, in forms that hang no GPU.

A rank that is absent must cost its peers an error, not a hang:
  - in the peer-memory form every device-side wait is bounded. Here one process plays rank 0 of a world of 2 whose
    "rank 1" is a set of buffers nobody serves, so the wait for rank 1's request runs out (after a deliberately small
    number of polls): the kernels return, a status word says which wait it was, the pass fails with a message, and
    the CUDA context stays usable;
  - in the NCCL form the communicator set-up is waited for with a limit: a world of 2 with only one rank present
    fails after the time-out instead of blocking for ever. No kernel is involved.
"""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture()
def be():
    from llamd_rs_b200 import backend

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    backend.stream_init()
    return backend


def test_a_wait_for_an_absent_rank_runs_out_and_reports(be):
    from llamd_rs_b200 import model as M
    from llamd_rs_b200 import synth

    hp = synth.TINY
    single = M.CudaModel.load_synthetic(hp, 5, max_kv=16)
    want = [single.forward(3, 0), single.forward(7, 1)]
    single.free()
    M.ep_init_local(0, 2)
    try:
        m = M.CudaModel.load_synthetic(hp, 5, max_kv=16)
        E, nu = hp["n_embd"], hp["n_expert_used"]
        own = m.ep_p2p_buffers()  # (this also fixes the prefill tile capacity)
        cap = m.ep_tile_cap()
        assert cap == 16  # min(prefill_tile, 40960 / (world * n_used), max_kv)
        # what rank 1 would have shared: expert outputs, arrival counter, gathered ids / scales / quants, dispatch counter,
        # then a prefill tile's expert outputs and gathered quants / scales / ids
        sizes = [nu * E * 4, 256, 2 * nu * 4, 2 * (E // 256) * 4, 2 * E, 256,
                 cap * nu * E * 4, 2 * cap * E, 2 * cap * (E // 256) * 4, 2 * cap * nu * 4]
        absent = [be.DevBuf.zeroed(n) for n in sizes]
        m.ep_p2p_attach_ptrs([own, [b.ptr for b in absent]])
        m.set_option("ep_poll_limit", 2000)  # a fraction of a millisecond per wait
        for use_graph in (True, False):
            m.use_graph = use_graph
            t0 = time.time()
            with pytest.raises(be.LlamdError) as err:
                m.forward(3, 0)
            assert time.time() - t0 < 5.0, "the bounded wait must give up quickly"
            assert "ran out" in str(err.value) and "recreated" in str(err.value)
            assert m.ep_status() == 2, "the first wait to run out is the one for the other rank's request"
        with pytest.raises(be.LlamdError) as err:
            m.prefill([3, 7, 9], 0)  # the tiled path waits for the absent rank's tile just the same
        assert "ran out" in str(err.value)
        m.free()
    finally:
        M.ep_finalize()
    # the context is intact: a fresh single-GPU model gives the same tokens as before
    again = M.CudaModel.load_synthetic(hp, 5, max_kv=16)
    assert [again.forward(3, 0), again.forward(7, 1)] == want
    again.free()


_CHILD = """
import sys, time
sys.path.insert(0, %r)
from llamd_rs_b200 import backend, model as M
backend.stream_init()
M.ep_set_timeout_ms(1500)
t0 = time.time()
try:
    M.ep_init(0, 2, lambda b: b)  # a world of two, and nobody else comes
    print("RESULT joined")
except backend.LlamdError as e:
    print("RESULT", round(time.time() - t0, 2), M._bind().llamd_cuda_ep_world(), str(e))
    M._bind().llamd_fwd_last_error()  # read and clear the sticky error, as a caller that goes on would
import numpy as np
print("ALIVE", backend.quantize_q8k_on_device(np.arange(256, dtype=np.float32))[0].size)
sys.stdout.flush()
import os
os._exit(0)  # the helper thread of the abandoned set-up is still inside NCCL's bootstrap
"""


def test_communicator_setup_gives_up_on_a_rank_that_never_joins(be):
    """In a child process: the abandoned set-up leaves a thread inside NCCL's bootstrap, which should not outlive the test."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
    out = subprocess.run([sys.executable, "-c", _CHILD % root], capture_output=True, text=True, timeout=300, env=env)
    lines = {l.split()[0]: l for l in out.stdout.splitlines() if l.startswith(("RESULT", "ALIVE"))}
    assert "RESULT" in lines and "ALIVE" in lines, (out.stdout[-1500:], out.stderr[-1500:])
    f = lines["RESULT"].split(None, 3)
    assert f[1] != "joined" and 1.0 < float(f[1]) < 30.0, lines["RESULT"]
    assert f[2] == "1", "a failed set-up leaves the process single-GPU"
    assert "never joined" in f[3]
    assert lines["ALIVE"].split()[1] == "256", "the device still answers"
