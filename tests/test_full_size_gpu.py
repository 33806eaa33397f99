"""The BASELINE configurations at their full sizes on the GPU, launched exactly as the benchmark launches them.

Each configuration goes to the device whole (256, 256, 256 and 160 (batch, head) problems in one call per
op), so the kernels take the same scheduling branch as in the timed runs: work items fetched from a counter,
problems walked in groups sized for L2. The CPU oracle needs about a second per problem at these sizes, so:

  * at least eight problems spread over the scheduling groups (the first and last of the batch, the two
    sides of a group boundary, others in between) are compared with the oracle, all three ops;
  * every problem of the full launch is compared bit for bit with the same problem computed in a launch of
    three problems, the shape of launch the oracle comparisons of tests/test_sdpa_gpu.py cover; one owner per
    output row and a fixed accumulation order make the bits independent of where a problem sits in a batch,
    so any difference is a mapping error;
  * with V set to ones every output row is a convex combination of ones: O == 1 for every row of every problem;
  * the row dot delta is compared directly with the oracle's;
  * two runs give the same bits.

Inputs are the benchmark's own seeded generators.
"""

from __future__ import annotations

import numpy as np
import pytest
from conftest import BF16, parity

from oracle import sdpa_oracle as oracle

pytestmark = pytest.mark.gpu

CONFIGS = ["gpt_layer", "prefill_4k", "encoder_2k", "ragged_3000"]


class FullRun:
    """One workload resident on the device at its full size, every op run once over the whole batch."""

    def __init__(self, workload: str, ones_v: bool = False, backward: bool = True):
        import bench
        from limn_b200 import runtime
        from limn_b200._lib import check, lib

        self.runtime, self.check, self.L = runtime, check, lib()
        b, h, s, d, causal, *_ = bench.WORKLOADS[workload]
        self.workload, self.bh, self.s, self.d, self.causal = workload, b * h, s, d, causal
        self.host = bench.shard_inputs(workload, 0, self.bh, True)
        if ones_v:
            self.host[2][...] = 1
        self.dev = [runtime.upload(a) for a in self.host]
        self.results = self.launch(self.dev, self.bh, backward)

    def launch(self, dev, bh, backward=True):
        """Forward (and delta, dQ, dK/dV) over `bh` problems whose operands start at the given buffers."""
        runtime, check, L, s, d = self.runtime, self.check, self.L, self.s, self.d
        q, k, v, do = (b.ptr if hasattr(b, "ptr") else b for b in dev)
        nbytes = bh * s * d * 2
        out, lse = runtime.empty(nbytes), runtime.empty(bh * s * 4)
        tail = (2, bh, s, s, d, d, int(self.causal), d**-0.5, None)
        check(L.limn_b200_sdpa_fwd(q, k, v, None, out.ptr, lse.ptr, *tail), "sdpa")
        found = {"out": (out, BF16, (bh, s, d)), "lse": (lse, np.float32, (bh, s))}
        if backward:
            delta, dq, dk, dv = runtime.empty(bh * s * 4), runtime.empty(nbytes), runtime.empty(nbytes), runtime.empty(nbytes)
            check(L.limn_b200_sdpa_delta(out.ptr, do, delta.ptr, 2, bh * s, d, None), "row dot")
            check(L.limn_b200_sdpa_bwd_q(q, k, v, do, lse.ptr, delta.ptr, None, dq.ptr, *tail), "sdpa_bwd_q")
            check(L.limn_b200_sdpa_bwd_kv(q, k, v, do, lse.ptr, delta.ptr, None, dk.ptr, dv.ptr, *tail), "sdpa_bwd_kv")
            found.update(delta=(delta, np.float32, (bh, s)), dq=(dq, BF16, (bh, s, d)), dk=(dk, BF16, (bh, s, d)), dv=(dv, BF16, (bh, s, d)))
        assert runtime.device_status() == 0
        return {name: runtime.download(buf, dtype, shape) for name, (buf, dtype, shape) in found.items()}

    def small_launch(self, first: int, count: int):
        """The same problems [first, first + count) as a launch of their own, read in place from the full buffers."""
        step = self.s * self.d * 2
        return self.launch([b.ptr + first * step for b in self.dev], count)


def spread(bh: int, group: int) -> list[int]:
    """Eight or more problems: both ends of the batch, both sides of the first and of a middle group boundary, and
    some in between."""
    middle = (bh // 2 // group) * group
    picks = {0, group - 1, group, middle - 1, middle, middle + group // 2, bh - group, bh - 1, bh // 3, (2 * bh) // 3 + 1}
    picks |= {(i * (bh - 1)) // 7 for i in range(8)}  # one group only (a small workload): evenly spaced instead
    return sorted(p for p in picks if 0 <= p < bh)


@pytest.mark.parametrize("workload", CONFIGS)
def test_the_benchmarked_launch_matches_the_oracle_and_small_launches(workload):
    run = FullRun(workload)
    got, s, d, causal, bh = run.results, run.s, run.d, run.causal, run.bh
    # the scheduling group of this launch, as the library picks it for the forward (capi.cu: work_group)
    streamed = s * 2 * d * 2
    group = max(1, min(bh, (32 << 20) // streamed))
    problems = spread(bh, group)
    assert len(problems) >= 8
    for p in problems:
        q, k, v, do = (a[p] for a in run.host)
        want_out, want_lse = oracle.sdpa_forward(q, k, v, causal=causal, scale=d**-0.5)
        tag = f"{workload}[{p} of {bh}]"
        parity(got["out"][p], want_out, 2e-2, f"{tag} O")
        parity(got["lse"][p], want_lse[..., 0], 1e-3, f"{tag} L")
        want_delta = oracle.row_delta(do, want_out)
        # delta from the device's own (rounded) O; the oracle's O may differ by a bfloat16 step, hence the bf16 tolerance scaled by |dO|
        parity(got["delta"][p], want_delta[..., 0], 2e-2, f"{tag} delta")
        want_dq = oracle.sdpa_backward_q(q, k, v, do, want_lse, want_delta, causal=causal, scale=d**-0.5)
        want_dk, want_dv = oracle.sdpa_backward_kv(q, k, v, do, want_lse, want_delta, causal=causal, scale=d**-0.5)
        for name, want in (("dq", want_dq), ("dk", want_dk), ("dv", want_dv)):
            parity(got[name][p], want, 2e-2, f"{tag} {name}")
    # every problem of the full launch against launches of three
    chunk = 3
    for first in range(0, bh, chunk):
        count = min(chunk, bh - first)
        small = run.small_launch(first, count)
        for name in ("out", "lse", "delta", "dq", "dk", "dv"):
            a, b = got[name][first:first + count], small[name]
            assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), f"{workload}: {name} of problems {first}..{first + count - 1} depends on the launch"


def test_delta_matches_the_oracle_row_dot_on_the_oracles_own_output():
    """limn_b200_sdpa_delta alone: fed the oracle's O, it must give the oracle's delta to float32 rounding."""
    from limn_b200 import runtime
    from limn_b200._lib import check, lib

    rng = np.random.default_rng(8)
    for dtype, code, shape in ((BF16, 2, (5, 300, 128)), (np.float16, 1, (3, 77, 64)), (np.float32, 0, (2, 50, 24))):
        out = rng.standard_normal(shape).astype(np.float32).astype(dtype)
        do = rng.standard_normal(shape).astype(np.float32).astype(dtype)
        rows = shape[0] * shape[1]
        delta, out_dev, do_dev = runtime.empty(rows * 4), runtime.upload(out), runtime.upload(do)
        check(lib().limn_b200_sdpa_delta(out_dev.ptr, do_dev.ptr, delta.ptr, code, rows, shape[2], None), "row dot")
        got = runtime.download(delta, np.float32, shape[:2])
        parity(got, oracle.row_delta(do, out)[..., 0], 1e-5, f"delta {np.dtype(dtype).name} {shape}")


@pytest.mark.parametrize("workload", ["prefill_4k", "ragged_3000", "encoder_2k"])
def test_rows_of_ones_come_back_as_ones_for_every_problem(workload):
    """softmax weights sum to 1, so V = 1 must give O = 1 in every row of every problem, ragged tail included."""
    run = FullRun(workload, ones_v=True, backward=False)
    out = run.results["out"].astype(np.float32)
    worst_per_problem = np.abs(out - 1.0).reshape(run.bh, -1).max(axis=1)
    assert worst_per_problem.max() <= 2**-7, f"problem {int(worst_per_problem.argmax())}"  # one bfloat16 step at 1.0
    assert np.isfinite(run.results["lse"]).all()


def test_full_size_runs_are_bit_identical():
    first = FullRun("ragged_3000").results
    second = FullRun("ragged_3000").results
    for key in ("out", "lse", "dq", "dk", "dv"):
        np.testing.assert_array_equal(first[key].view(np.uint8), second[key].view(np.uint8))


def test_operands_past_2_31_elements():
    """The largest case: 520 problems of 32 768 tokens at head dim 128, 2.18e9 elements (4.4 GB) per operand, so that
    element offsets no longer fit 32 bits and a problem's tiles lie 8 MB apart. Q, K and dO repeat a seeded block of 8
    problems; V is that block times a per-problem constant, so a problem that read its neighbour's tiles would show.
    Rows of O, L, dQ, dK and dV sampled over the batch (its first and last problems and the three around the 2^31st
    element) are compared with a row-wise numpy evaluation of limn/sdpa.py:114-203, which needs one row's scores at a
    time instead of the 4 GB score matrix of a problem."""
    torch = pytest.importorskip("torch")
    from limn_b200 import runtime
    from limn_b200._lib import check, lib

    L = lib()
    block, bh, s, d = 8, 520, 32768, 128
    assert bh * s * d > 2**31
    scale = d**-0.5
    rng = np.random.default_rng(2031)
    base = [(rng.standard_normal((block, s, d), dtype=np.float32) * m).astype(BF16) for m in (0.5, 0.5, 1.0, 1.0)]
    consts = 0.25 * (1 + np.arange(bh) % 7)
    dev = torch.device("cuda", 0)
    runtime.set_device(0)
    on_device = [torch.from_numpy(a.view(np.int16)).to(dev).view(torch.bfloat16) for a in base]
    q, k, vb, do = (t.repeat(bh // block, 1, 1) for t in on_device)
    v = (vb.float() * torch.from_numpy(consts.astype(np.float32)).to(dev)[:, None, None]).to(torch.bfloat16)
    del vb
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    lse, delta = (torch.empty((bh, s), dtype=torch.float32, device=dev) for _ in range(2))
    tail = (2, bh, s, s, d, d, 1, scale, None)
    check(L.limn_b200_sdpa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, out.data_ptr(), lse.data_ptr(), *tail), "sdpa")
    check(L.limn_b200_sdpa_bwd_q_fused(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), do.data_ptr(), lse.data_ptr(), None,
                                       dq.data_ptr(), delta.data_ptr(), *tail), "sdpa_bwd_q")
    check(L.limn_b200_sdpa_bwd_kv(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(), None,
                                  dk.data_ptr(), dv.data_ptr(), *tail), "sdpa_bwd_kv")
    torch.cuda.synchronize()
    assert runtime.device_status() == 0

    f32 = lambda a: a.astype(np.float32)
    host = lambda t, p, rows: t[p, rows].float().cpu().numpy()
    edge = -(-(2**31) // (s * d))  # the first problem that starts past the 2^31st element
    for p in (0, 1, edge - 1, edge, edge + 1, bh - 1):
        qb, kb, dob = (f32(a[p % block]) for a in (base[0], base[1], base[3]))
        vp = f32((f32(base[2][p % block]) * np.float32(consts[p])).astype(BF16))  # V as the device holds it
        rows = [0, 1, 127, 128, 4095, 20000, s - 1]
        want_o, want_l, want_dq = [], [], []
        for i in rows:
            sc = (kb[: i + 1] @ qb[i]) * scale
            top = sc.max()
            w = np.exp(sc - top)
            den = w.sum()
            o = (w @ vp[: i + 1]) / den
            want_o.append(o)
            want_l.append(top + np.log(den))
            dp = vp[: i + 1] @ dob[i]
            ds = (w / den) * (dp - dob[i] @ o) * scale
            want_dq.append(ds @ kb[: i + 1])
        parity(host(out, p, rows), np.array(want_o, np.float32), 2e-2, f"problem {p} O")
        parity(host(lse, p, rows), np.array(want_l, np.float32), 1e-3, f"problem {p} L")
        parity(host(dq, p, rows), np.array(want_dq, np.float32), 2e-2, f"problem {p} dQ")
        # dK and dV of late keys: only the last queries see them, and the device's L and delta for those rows are
        # what the kernels read (L was checked above on a sample of the same rows' neighbours)
        first = s - 300
        li = lse[p, first:].cpu().numpy()
        di = delta[p, first:].cpu().numpy()
        keys = [first, s - 129, s - 128, s - 1]
        want_dk, want_dv = [], []
        for j in keys:
            i0 = j - first
            sc = (qb[j:] @ kb[j]) * scale
            pj = np.exp(sc - li[i0:])
            want_dv.append(pj @ dob[j:])
            dpj = dob[j:] @ vp[j]
            want_dk.append((pj * (dpj - di[i0:]) * scale) @ qb[j:])
        parity(host(dk, p, keys), np.array(want_dk, np.float32), 2e-2, f"problem {p} dK")
        parity(host(dv, p, keys), np.array(want_dv, np.float32), 2e-2, f"problem {p} dV")
