"""The allocation-free attention entry point against the regular one.

``llamd_fwd_attention_noalloc`` serves hosts that may not allocate device
memory at call time (a serving process whose own pool owns the GPU, a loop that
cannot afford the allocator's device synchronisation): its score scratch is an
array built into the library. It must give bit for bit what
``llamd_fwd_attention`` gives with a caller-supplied scratch buffer, on two
calls in a row (the second finds the first call's scores still in the array),
and it must refuse shapes beyond the array.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run_both(backend, lib, synth, n_kv, seed, check_free=False):
    n_head, n_head_kv, hd = 32, 4, 128
    q = synth.normal_f32(n_head * hd, seed, "na.q")
    k = synth.normal_f32(n_kv * n_head_kv * hd, seed, "na.k")
    v = synth.normal_f32(n_kv * n_head_kv * hd, seed, "na.v")
    dq, dk, dv = backend.DevBuf.from_array(q), backend.DevBuf.from_array(k), backend.DevBuf.from_array(v)
    want_buf, got_buf = backend.DevBuf(q.nbytes), backend.DevBuf.zeroed(q.nbytes)
    scores = backend.DevBuf(n_head * n_kv * 4)
    lib.llamd_fwd_attention(dq.ptr, dk.ptr, dv.ptr, want_buf.ptr, scores.ptr, n_head, n_head_kv, hd, n_kv)
    backend.sync()
    want = want_buf.download_f32(q.size)
    free_before = backend.free_memory()
    rc = lib.llamd_fwd_attention_noalloc(dq.ptr, dk.ptr, dv.ptr, got_buf.ptr, n_head, n_head_kv, hd, n_kv)
    assert rc == 0, backend._last_error()
    backend.sync()
    if check_free:
        assert backend.free_memory() == free_before, "a warmed-up call must take no device memory"
    got = got_buf.download_f32(q.size)
    assert np.all(np.isfinite(want)) and np.any(want != 0)
    return got, want


def test_noalloc_attention_matches_the_regular_entry_point_twice():
    from llamd_rs_b200 import backend, synth
    from llamd_rs_b200._lib import lib

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    backend.stream_init()
    L = lib()
    # two calls in a row; the second is shorter, so stale scores of the first sit beyond (and under) it
    for i, (n_kv, seed) in enumerate(((700, 1), (133, 2))):
        got, want = run_both(backend, L, synth, n_kv, seed, check_free=i > 0)  # the first call may load code and resolve the array
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"n_kv={n_kv}: differs from llamd_fwd_attention"


def test_noalloc_attention_refuses_more_than_its_scratch():
    from llamd_rs_b200 import backend
    from llamd_rs_b200._lib import lib

    if not backend.available():
        pytest.fail("no CUDA device: the GPU tests must run on a GPU box")
    backend.stream_init()
    L = lib()
    tiny = backend.DevBuf(64)
    # 64 heads x 4097 positions is one row too many; refused before any launch, so the small buffers are never read
    rc = L.llamd_fwd_attention_noalloc(tiny.ptr, tiny.ptr, tiny.ptr, tiny.ptr, 64, 4, 128, 4097)
    assert rc == -1 and "262144" in backend._last_error()
    L.llamd_fwd_last_error()  # clear the sticky flag for whoever runs next
    assert L.llamd_fwd_attention_noalloc(None, tiny.ptr, tiny.ptr, tiny.ptr, 4, 4, 128, 1) == -1
    L.llamd_fwd_last_error()
    # 4 heads x 60000 positions fits the array but not the shared-memory score row: refused, and the message says which limit
    rc = L.llamd_fwd_attention_noalloc(tiny.ptr, tiny.ptr, tiny.ptr, tiny.ptr, 4, 4, 128, 60000)
    assert rc == -1 and "shared-memory" in backend._last_error()
    L.llamd_fwd_last_error()
    # while an earlier error is unread the call launches nothing and says so through its return value
    assert L.llamd_fwd_attention_noalloc(None, tiny.ptr, tiny.ptr, tiny.ptr, 4, 4, 128, 1) == -1
    assert L.llamd_fwd_attention_noalloc(tiny.ptr, tiny.ptr, tiny.ptr, tiny.ptr, 4, 4, 128, 1) == -1
    L.llamd_fwd_last_error()
