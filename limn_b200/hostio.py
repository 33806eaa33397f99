"""Attention over tensors that live in host memory: upload, compute and download overlapped.

limn keeps tensors on the device between steps, so its own path never needs this. A host
that holds Q, K, V (and dO) in pinned memory and wants O, L (and dQ, dK, dV) back in pinned
memory pays for the PCIe transfers either way; what it need not pay for is waiting for them
one after the other. The (batch, head) problems are independent, so `HostPipeline` cuts the
batch into chunks and runs three streams: one uploads chunk i+1 while a second runs the
kernels on chunk i and a third downloads chunk i-1. Two sets of device buffers are enough,
and their size is set by the chunk, not by the batch, so a batch larger than device memory
works too. The kernels are the same ones the registry builders launch; nothing here
computes.
"""

from __future__ import annotations

import numpy as np

from limn_b200 import runtime
from limn_b200._lib import DTYPE_CODES, check, lib


class HostPipeline:
    """forward (and optionally backward) of `bh` problems of shape (t, d), 16-bit storage, host to host.

    Arguments are numpy arrays over pinned memory (`runtime.PinnedArray(...).array`), shaped
    (bh, t, d) for Q, K, V, dO, O, dQ, dK, dV and (bh, t) float32 for L. `chunk` problems are
    in flight per stage; by default the batch is cut into at least eight chunks (of at most 16
    problems), so that upload, kernels and download overlap even when the batch is small.
    """

    def __init__(self, bh: int, t: int, d: int, *, dtype: str = "bfloat16", causal: bool, backward: bool, chunk: int | None = None):
        if dtype not in ("bfloat16", "float16"):
            raise ValueError("HostPipeline moves 16-bit storage; other dtypes go through the registry builders")
        self.bh, self.t, self.d, self.causal, self.backward = bh, t, d, causal, backward
        self.code = DTYPE_CODES[dtype]
        self.scale = d ** -0.5
        if chunk is None:
            chunk = min(16, -(-bh // 8))
        self.chunk = max(1, min(chunk, bh))
        self.row_bytes = t * d * 2
        self.lib = lib()
        self.up, self.run, self.down = runtime.Stream(), runtime.Stream(), runtime.Stream()
        inputs = 4 if backward else 3
        outputs = 4 if backward else 1  # O (+ dQ, dK, dV); L and delta are separate
        self.sets = []
        for _ in range(2):
            tensors = [runtime.empty(self.chunk * self.row_bytes, poison=None) for _ in range(inputs + outputs)]
            stats = [runtime.empty(self.chunk * t * 4, poison=None) for _ in range(2)]  # L, delta
            events = {name: runtime.Event() for name in ("uploaded", "computed", "free")}
            self.sets.append((tensors[:inputs], tensors[inputs:], stats, events))
        self.launches = 0

    def _check(self, code: int, doing: str) -> None:
        check(code, doing)

    def __call__(self, q, k, v, out, lse, do=None, dq=None, dk=None, dv=None) -> tuple[int, int]:
        """Enqueue the whole batch and wait for it. Returns (bytes uploaded, bytes downloaded)."""
        L, t, d = self.lib, self.t, self.d
        host_in = [q, k, v] + ([do] if self.backward else [])
        host_out = [out] + ([dq, dk, dv] if self.backward else [])
        up_bytes = down_bytes = 0
        self.launches = 0
        used = [False, False]
        for index, first in enumerate(range(0, self.bh, self.chunk)):
            count = min(self.chunk, self.bh - first)
            ins, outs, (lse_dev, delta_dev), events = self.sets[index % 2]
            nbytes = count * self.row_bytes
            # upload, once the previous user of this buffer set has been downloaded
            if used[index % 2]:
                self.up.wait(events["free"])
            for src, dst in zip(host_in, ins):
                self._check(L.limn_b200_copy_h2d(dst.ptr, src[first:first + count].ctypes.data, nbytes, self.up.handle), "uploading a chunk")
                up_bytes += nbytes
            events["uploaded"].record(self.up)
            # compute
            self.run.wait(events["uploaded"])
            tail = (self.code, count, t, t, d, d, int(self.causal), self.scale, self.run.handle)
            qd, kd, vd = (b.ptr for b in ins[:3])
            self._check(L.limn_b200_sdpa_fwd(qd, kd, vd, None, outs[0].ptr, lse_dev.ptr, *tail), "sdpa")
            self.launches += L.limn_b200_last_launch_count()
            if self.backward:
                dod = ins[3].ptr
                self._check(L.limn_b200_sdpa_bwd_q_fused(qd, kd, vd, outs[0].ptr, dod, lse_dev.ptr, None, outs[1].ptr, delta_dev.ptr, *tail), "sdpa_bwd_q")
                self.launches += L.limn_b200_last_launch_count()
                self._check(L.limn_b200_sdpa_bwd_kv(qd, kd, vd, dod, lse_dev.ptr, delta_dev.ptr, None, outs[2].ptr, outs[3].ptr, *tail), "sdpa_bwd_kv")
                self.launches += L.limn_b200_last_launch_count()
            events["computed"].record(self.run)
            # download
            self.down.wait(events["computed"])
            for dst, src in zip(host_out, outs):
                self._check(L.limn_b200_copy_d2h(dst[first:first + count].ctypes.data, src.ptr, nbytes, self.down.handle), "downloading a chunk")
                down_bytes += nbytes
            stat_bytes = count * t * 4
            self._check(L.limn_b200_copy_d2h(lse[first:first + count].ctypes.data, lse_dev.ptr, stat_bytes, self.down.handle), "downloading L")
            down_bytes += stat_bytes
            events["free"].record(self.down)
            used[index % 2] = True
        self.down.synchronize()
        self.run.synchronize()
        self.up.synchronize()
        return up_bytes, down_bytes


def pinned_like(array: np.ndarray) -> runtime.PinnedArray:
    """A pinned copy of `array` (keep the returned object alive as long as its `.array` is used)."""
    holder = runtime.PinnedArray(array.shape, array.dtype if array.dtype.itemsize != 2 else np.uint16)
    holder.array[...] = array.view(holder.array.dtype) if array.dtype.itemsize == 2 else array
    return holder
