"""The BASELINE configurations at their full sizes on the GPU.

The CPU oracle needs about half a second per (batch, head) problem at these sizes, so each
configuration is checked on a few problems picked across the batch (first, last, one inside),
all three ops, plus two size-independent properties over the whole tensor: with V set to ones
every output row is exactly a convex combination of ones (O == 1), and two runs give the same
bits. Inputs are the benchmark's own seeded generators."""

from __future__ import annotations

import numpy as np
import pytest
from conftest import BF16

from oracle import sdpa_oracle as oracle

pytestmark = pytest.mark.gpu

CONFIGS = ["gpt_layer", "prefill_4k", "encoder_2k", "ragged_3000"]


def _device_run(workload, problems, ones_v=False):
    import bench
    from limn_b200 import runtime
    from limn_b200._lib import check, lib

    L = lib()
    b, h, s, d, causal, backward, *_ = bench.WORKLOADS[workload]
    bh = len(problems)
    host = [np.empty((bh, s, d), dtype=BF16) for _ in range(4)]
    for i, problem in enumerate(problems):
        for dst, src in zip(host, bench.problem_inputs(workload, problem)):
            dst[i] = src
    if ones_v:
        host[2][...] = 1
    q, k, v, do = (runtime.upload(a) for a in host)
    nbytes = bh * s * d * 2
    out, lse, delta = runtime.empty(nbytes), runtime.empty(bh * s * 4), runtime.empty(bh * s * 4)
    tail = (2, bh, s, s, d, d, int(causal), d**-0.5, None)
    check(L.limn_b200_sdpa_fwd(q.ptr, k.ptr, v.ptr, None, out.ptr, lse.ptr, *tail), "sdpa")
    result = {"inputs": host, "out": runtime.download(out, BF16, (bh, s, d)), "lse": runtime.download(lse, np.float32, (bh, s))}
    if backward and not ones_v:
        dq, dk, dv = (runtime.empty(nbytes) for _ in range(3))
        check(L.limn_b200_sdpa_delta(out.ptr, do.ptr, delta.ptr, 2, bh * s, d, None), "row dot")
        check(L.limn_b200_sdpa_bwd_q(q.ptr, k.ptr, v.ptr, do.ptr, lse.ptr, delta.ptr, None, dq.ptr, *tail), "sdpa_bwd_q")
        check(L.limn_b200_sdpa_bwd_kv(q.ptr, k.ptr, v.ptr, do.ptr, lse.ptr, delta.ptr, None, dk.ptr, dv.ptr, *tail), "sdpa_bwd_kv")
        for name, buf in (("dq", dq), ("dk", dk), ("dv", dv)):
            result[name] = runtime.download(buf, BF16, (bh, s, d))
    assert runtime.device_status() == 0
    return result


@pytest.mark.parametrize("workload", CONFIGS)
def test_sampled_problems_match_the_oracle_at_full_size(workload):
    import bench

    b, h, s, d, causal, backward, *_ = bench.WORKLOADS[workload]
    bh = b * h
    problems = [0, bh // 2 + 1, bh - 1]
    got = _device_run(workload, problems)
    for i in range(len(problems)):
        q, k, v, do = (a[i] for a in got["inputs"])
        want_out, want_lse = oracle.sdpa_forward(q, k, v, causal=causal, scale=d**-0.5)
        assert oracle.worst(got["out"][i].astype(np.float32), want_out.astype(np.float32)) <= 2e-2
        assert float(np.abs(got["lse"][i] - want_lse[..., 0]).max()) <= 1e-3
        if backward:
            delta = oracle.row_delta(do, want_out)
            want_dq = oracle.sdpa_backward_q(q, k, v, do, want_lse, delta, causal=causal, scale=d**-0.5)
            want_dk, want_dv = oracle.sdpa_backward_kv(q, k, v, do, want_lse, delta, causal=causal, scale=d**-0.5)
            for name, want in (("dq", want_dq), ("dk", want_dk), ("dv", want_dv)):
                err = oracle.worst(got[name][i].astype(np.float32), want.astype(np.float32))
                assert err <= 2e-2, f"{workload} problem {problems[i]} {name}: {err:.3e}"


@pytest.mark.parametrize("workload", ["prefill_4k", "ragged_3000"])
def test_rows_of_ones_come_back_as_ones(workload):
    """softmax weights sum to 1, so V = 1 must give O = 1 in every row, ragged tail included."""
    import bench

    b, h = bench.WORKLOADS[workload][:2]
    got = _device_run(workload, list(range(0, b * h, max(1, b * h // 16))), ones_v=True)
    out = got["out"].astype(np.float32)
    assert np.abs(out - 1.0).max() <= 2**-7  # one bfloat16 step at 1.0
    assert np.isfinite(got["lse"]).all()


def test_full_size_runs_are_bit_identical():
    first = _device_run("ragged_3000", [3, 77])
    second = _device_run("ragged_3000", [3, 77])
    for key in ("out", "lse", "dq", "dk", "dv"):
        np.testing.assert_array_equal(first[key].view(np.uint8), second[key].view(np.uint8))
