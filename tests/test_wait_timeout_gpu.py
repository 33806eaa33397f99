"""The give-up path of the bounded waits, walked end to end without hanging or faulting anything.

Every wait in the tensor-core kernels (on a TMA copy, on the tensor pipe, on another warp) is bounded: when
its budget runs out the kernel records 0x5741rrbb in the device's status word and returns, and kernels that
start while the word is set stand down at once. limn_b200_wait_probe makes exactly that happen with a
one-warp kernel of its own that waits a few microseconds on a barrier nobody arrives at; the production
kernels are not touched. The test then checks what the rest of the library promises about that state."""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
from conftest import BF16

pytestmark = pytest.mark.gpu


def _forward(L, check, runtime, q, k, v, shape, poison=0xFF):
    bh, t, d = shape
    out, lse = runtime.empty(bh * t * d * 2, poison=poison), runtime.empty(bh * t * 4, poison=poison)
    check(L.limn_b200_sdpa_fwd(q.ptr, k.ptr, v.ptr, None, out.ptr, lse.ptr, 2, bh, t, t, d, d, 1, d**-0.5, None), "sdpa")
    return out, lse


def test_a_wait_that_runs_out_is_reported_and_the_device_recovers():
    from limn_b200 import runtime
    from limn_b200._lib import DEVICE_TIMEOUT, check, last_error, lib

    L = lib()
    runtime.set_device(0)
    assert runtime.device_status() == 0
    shape = (40, 300, 128)  # 120 work items: enough CTAs to show that every one of them stands down
    rng = np.random.default_rng(31)
    q, k, v = (runtime.upload(rng.standard_normal(shape).astype(np.float32).astype(BF16)) for _ in range(3))
    out, lse = _forward(L, check, runtime, q, k, v, shape)
    good = runtime.download(out, np.uint16, shape), runtime.download(lse, np.uint32, shape[:2])

    # 1. the wait runs out: status code in the word, the probe's own flag says it gave up, the kernel returned
    gave_up = runtime.empty(4, poison=0)
    check(L.limn_b200_wait_probe(20000, gave_up.ptr, None), "wait probe")
    # 2. a production launch enqueued while the word is set writes nothing
    out2, lse2 = _forward(L, check, runtime, q, k, v, shape, poison=0xAB)
    runtime.synchronize()
    assert runtime.download(gave_up, np.uint32, (1,))[0] == 1
    assert (runtime.download(out2, np.uint8, (out2.nbytes,)) == 0xAB).all(), "a kernel ran although an earlier one had given up"
    assert (runtime.download(lse2, np.uint8, (lse2.nbytes,)) == 0xAB).all()
    # 3. the word is read as an error, once
    word = ctypes.c_uint(0)
    assert L.limn_b200_device_status(ctypes.byref(word)) == DEVICE_TIMEOUT
    assert word.value == 0x57417E57
    assert "gave up on a bounded wait" in last_error() and "57417e57" in last_error()
    assert L.limn_b200_device_status(ctypes.byref(word)) == 0 and word.value == 0
    # 4. and the next launches are right again: the aborted launch left its work counters at zero
    for _ in range(3):
        out3, lse3 = _forward(L, check, runtime, q, k, v, shape)
        np.testing.assert_array_equal(runtime.download(out3, np.uint16, shape), good[0])
        np.testing.assert_array_equal(runtime.download(lse3, np.uint32, shape[:2]), good[1])
    assert runtime.device_status() == 0


def test_finish_raises_like_a_failed_kernel_of_the_reference():
    """limn_b200.install() wraps the device's finish(): after a batch in which one of our Runners ran, a set
    status word surfaces as RuntimeError("cuda: ..."), where limn raises for a failed kernel of its own."""
    import limn_b200
    from limn_b200 import registry, runtime
    from limn_b200._lib import check, lib

    class Device:
        def __init__(self):
            self.custom = {}
            self.synchronised = 0

        def finish(self):
            runtime.synchronize()
            self.synchronised += 1

    dev = limn_b200.install(Device())
    dev.finish()  # nothing of ours ran: no status read, nothing raised
    check(lib().limn_b200_wait_probe(5000, None, None), "wait probe")
    dev.finish()  # still nothing of ours in the batch: the word is not even looked at
    registry._note_launch()  # what every Runner does
    with pytest.raises(RuntimeError, match=r"cuda: waiting for the batch: a limn_b200 kernel gave up on a bounded wait \(status 0x57417e57\)"):
        dev.finish()
    dev.finish()
    assert dev.synchronised == 4 and runtime.device_status() == 0
