"""The allocation-free dQ entry point, limn_b200_sdpa_bwd_q_static, against the ordinary one.

It serves hosts that cannot allocate device memory (their own pool owns all of it, or they run
where CUDA's allocation calls are not allowed): delta and the kernels' status word come out of
a fixed array inside the library instead. The check is that it gives what limn_b200_sdpa_delta
followed by limn_b200_sdpa_bwd_q gives, on two calls in a row that share that array, the
second with different shapes so that anything left over from the first would show.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test."""

from __future__ import annotations

import ctypes

import ml_dtypes
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
BF16 = np.dtype(ml_dtypes.bfloat16)


def _both_ways(dtype, code, shape, causal, seed, masked=False, own_stream=False, want_status=True):
    from limn_b200 import runtime
    from limn_b200._lib import check, lib

    L = lib()
    bh, t, d = shape
    rng = np.random.default_rng(seed)
    q, k, v, do = (rng.standard_normal(shape).astype(np.float32).astype(dtype) for _ in range(4))
    stat = 4
    dq_, k_, v_, do_ = (runtime.upload(a) for a in (q, k, v, do))
    mask = None
    if masked:  # the last third of every problem's keys hidden, as a padded batch arrives
        mask = runtime.upload(np.broadcast_to(np.arange(t) < t * 2 // 3, (bh, t)).astype(np.float32).astype(dtype))
    mask_ptr = mask.ptr if mask is not None else None
    stream = runtime.Stream() if own_stream else None
    handle = stream.handle if stream is not None else None
    out, lse, delta = runtime.empty(q.nbytes), runtime.empty(bh * t * stat), runtime.empty(bh * t * stat)
    tail = (code, bh, t, t, d, d, int(causal), d**-0.5, None)
    check(L.limn_b200_sdpa_fwd(dq_.ptr, k_.ptr, v_.ptr, mask_ptr, out.ptr, lse.ptr, *tail), "sdpa")
    # the ordinary route: the caller owns delta
    want = runtime.empty(q.nbytes)
    check(L.limn_b200_sdpa_delta(out.ptr, do_.ptr, delta.ptr, code, bh * t, d, None), "row dot")
    check(L.limn_b200_sdpa_bwd_q(dq_.ptr, k_.ptr, v_.ptr, do_.ptr, lse.ptr, delta.ptr, mask_ptr, want.ptr, *tail), "sdpa_bwd_q")
    # the allocation-free route: inputs and outputs only
    got = runtime.empty(q.nbytes)
    status = runtime.empty(4) if want_status else None
    runtime.synchronize()  # a stream of the caller's own does not wait for the default stream by itself
    check(L.limn_b200_sdpa_bwd_q_static(dq_.ptr, k_.ptr, v_.ptr, out.ptr, do_.ptr, lse.ptr, mask_ptr, got.ptr,
                                        status.ptr if status is not None else None, *tail[:-1], handle),
          "sdpa_bwd_q_static")
    assert L.limn_b200_last_launch_count() == 2  # the row dot and the dQ kernel
    if stream is not None:
        stream.synchronize()
    runtime.synchronize()
    if status is not None:
        assert runtime.download(status, np.uint32, (1,))[0] == 0
    return runtime.download(got, dtype, shape), runtime.download(want, dtype, shape)


def test_static_dq_matches_the_ordinary_entry_point_twice_in_a_row():
    cases = [
        (BF16, 2, (3, 384, 128), True, 21, {}),    # tensor-core kernel, three tiles
        (BF16, 2, (2, 200, 64), False, 22, {}),    # smaller and ragged: stale delta rows from the first call lie beyond it
        (np.float32, 0, (2, 100, 32), True, 23, {}),  # the general kernel takes the same route
        (BF16, 2, (2, 300, 64), True, 24, {"masked": True}),                      # a key mask rides along
        (BF16, 2, (2, 260, 128), False, 25, {"own_stream": True, "want_status": False}),  # a stream of the caller's, no status word wanted
    ]
    for dtype, code, shape, causal, seed, how in cases:
        got, want = _both_ways(dtype, code, shape, causal, seed, **how)
        assert not np.isnan(got.astype(np.float32)).any()
        # same kernels over the same delta: the tolerance of the other parity tests is far more than needed
        np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), rtol=0, atol=2e-2 if dtype == BF16 else 1e-4)
        np.testing.assert_array_equal(got.view(np.uint8), want.view(np.uint8))


def test_static_dq_refuses_more_rows_than_its_array_holds():
    from limn_b200._lib import lib

    L = lib()
    one = 256  # never dereferenced: the size check comes first
    rows_too_many = (1 << 20) // 4096 + 1
    code = L.limn_b200_sdpa_bwd_q_static(one, one, one, one, one, one, None, one, None, 2, rows_too_many, 4096, 4096, 128, 128, 1,
                                         128**-0.5, None)
    assert code == 2
    message = L.limn_b200_last_error().decode()
    assert "exceed" in message and "1048576" in message
    assert L.limn_b200_sdpa_bwd_q_static(one, one, one, None, one, one, None, one, None, 2, 1, 4, 4, 8, 8, 0, 1.0, None) == 1


def test_a_refused_static_call_enqueues_nothing():
    """Every argument check comes before the first thing put on the stream: no kernel is counted for a refused
    call, whatever is wrong with it, and the status is the one for bad arguments, not a CUDA error."""
    from limn_b200 import runtime
    from limn_b200._lib import lib

    L = lib()
    buf = runtime.empty(1 << 16)
    p = buf.ptr
    refused = {
        "unknown dtype": (p, p, p, p, p, p, None, p, None, 9, 1, 8, 8, 64, 64, 0, 0.125, None),
        "null q": (None, p, p, p, p, p, None, p, None, 2, 1, 8, 8, 64, 64, 0, 0.125, None),
        "null lse": (p, p, p, p, p, None, None, p, None, 2, 1, 8, 8, 64, 64, 0, 0.125, None),
        "null dq": (p, p, p, p, p, p, None, None, None, 2, 1, 8, 8, 64, 64, 0, 0.125, None),
        "causal and rectangular": (p, p, p, p, p, p, None, p, None, 2, 1, 8, 9, 64, 64, 1, 0.125, None),
        "hd_v of zero": (p, p, p, p, p, p, None, p, None, 2, 1, 8, 8, 64, 0, 0, 0.125, None),
        "hd of zero": (p, p, p, p, p, p, None, p, None, 0, 1, 8, 8, 0, 8, 0, 0.125, None),
    }
    for why, args in refused.items():
        assert L.limn_b200_sdpa_bwd_q_static(*args) == 1, why
        assert L.limn_b200_last_launch_count() == 0, why
        assert L.limn_b200_last_error()
    assert runtime.device_status() == 0
