"""limn_b200.hostio.HostPipeline: host-to-host attention with the copies overlapped gives what the
plain device-resident calls give, bit for bit (same kernels, same inputs), for a batch that does not
divide into whole chunks."""

from __future__ import annotations

import ml_dtypes
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
BF16 = np.dtype(ml_dtypes.bfloat16)


@pytest.mark.parametrize("backward", [False, True], ids=["forward", "forward+backward"])
def test_pipeline_matches_device_resident_calls(backward):
    import limn_standin as host
    from limn_b200 import runtime
    from limn_b200.hostio import HostPipeline

    bh, t, d = 11, 300, 64
    rng = np.random.default_rng(5)
    q, k, v, do = (rng.standard_normal((bh, t, d)).astype(np.float32).astype(BF16) for _ in range(4))
    pinned = {}

    def pin(name, array=None, shape=None, dtype=None):
        holder = runtime.PinnedArray(array.shape if array is not None else shape, np.uint16 if dtype is None else dtype)
        if array is not None:
            holder.array[...] = array.view(np.uint16)
        pinned[name] = holder
        return holder.array

    args = [pin("q", q), pin("k", k), pin("v", v), pin("out", shape=(bh, t, d)), pin("lse", shape=(bh, t), dtype=np.float32)]
    extra = {}
    if backward:
        extra = dict(do=pin("do", do), dq=pin("dq", shape=(bh, t, d)), dk=pin("dk", shape=(bh, t, d)), dv=pin("dv", shape=(bh, t, d)))
    pipe = HostPipeline(bh, t, d, causal=True, backward=backward, chunk=4)
    up, down = pipe(*args, **extra)
    assert up == (4 if backward else 3) * bh * t * d * 2
    assert down == (4 if backward else 1) * bh * t * d * 2 + bh * t * 4
    assert pipe.launches == (3 if backward else 1) * 3  # three chunks, the row dot inside the dQ pass
    assert runtime.device_status() == 0

    att = host.Attention(host.Device(), q, k, v, causal=True)
    want_out, want_lse = att.forward()
    np.testing.assert_array_equal(pinned["out"].array, want_out.view(np.uint16))
    np.testing.assert_array_equal(pinned["lse"].array, want_lse[..., 0])
    if backward:
        # the pipeline computes the row dot inside the dQ pass, the comparison run as a kernel of its own: the two
        # sums differ in their last float32 bits, so the gradients agree to a bfloat16 step rather than bit for bit
        for name, want in zip(("dq", "dk", "dv"), att.backward(do)):
            got = pinned[name].array.view(BF16).astype(np.float32)
            np.testing.assert_allclose(got, want.astype(np.float32), rtol=2**-7, atol=2e-3)
