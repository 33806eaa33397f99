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


def _both_ways(dtype, code, shape, causal, seed):
    from limn_b200 import runtime
    from limn_b200._lib import check, lib

    L = lib()
    bh, t, d = shape
    rng = np.random.default_rng(seed)
    q, k, v, do = (rng.standard_normal(shape).astype(np.float32).astype(dtype) for _ in range(4))
    stat = 4
    dq_, k_, v_, do_ = (runtime.upload(a) for a in (q, k, v, do))
    out, lse, delta = runtime.empty(q.nbytes), runtime.empty(bh * t * stat), runtime.empty(bh * t * stat)
    tail = (code, bh, t, t, d, d, int(causal), d**-0.5, None)
    check(L.limn_b200_sdpa_fwd(dq_.ptr, k_.ptr, v_.ptr, None, out.ptr, lse.ptr, *tail), "sdpa")
    # the ordinary route: the caller owns delta
    want = runtime.empty(q.nbytes)
    check(L.limn_b200_sdpa_delta(out.ptr, do_.ptr, delta.ptr, code, bh * t, d, None), "row dot")
    check(L.limn_b200_sdpa_bwd_q(dq_.ptr, k_.ptr, v_.ptr, do_.ptr, lse.ptr, delta.ptr, None, want.ptr, *tail), "sdpa_bwd_q")
    # the allocation-free route: inputs and outputs only
    got = runtime.empty(q.nbytes)
    status = runtime.empty(4)
    check(L.limn_b200_sdpa_bwd_q_static(dq_.ptr, k_.ptr, v_.ptr, out.ptr, do_.ptr, lse.ptr, None, got.ptr, status.ptr, *tail),
          "sdpa_bwd_q_static")
    assert L.limn_b200_last_launch_count() == 2  # the row dot and the dQ kernel
    runtime.synchronize()
    assert runtime.download(status, np.uint32, (1,))[0] == 0
    return runtime.download(got, dtype, shape), runtime.download(want, dtype, shape)


def test_static_dq_matches_the_ordinary_entry_point_twice_in_a_row():
    cases = [
        (BF16, 2, (3, 384, 128), True, 21),    # tensor-core kernel, three tiles
        (BF16, 2, (2, 200, 64), False, 22),    # smaller and ragged: stale delta rows from the first call lie beyond it
        (np.float32, 0, (2, 100, 32), True, 23),  # the general kernel takes the same route
    ]
    for dtype, code, shape, causal, seed in cases:
        got, want = _both_ways(dtype, code, shape, causal, seed)
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
