"""Test scaffolding: a minimal host for the three ops, shaped like the parts of limn the kernels touch.

limn itself is the host: `limn_b200.install(limn.device.active())` and everything else is
limn's (tests/test_limn_dropin_gpu.py drives exactly that). This module lets the per-kernel
parity tests hand the registry builders nodes and buffers without going through limn's
frontend, so that they can poison outputs, pick odd shapes and read intermediate buffers: it
mirrors, by name and meaning,
  * DType / the four float dtypes and `accumulate_in` (limn/ops.py:18-27, :53-62),
  * `Custom` and `custom()`: one node per output, siblings sharing srcs (limn/ops.py:108-136),
  * a device with the `custom` registry, `has_custom`, `custom_runner` (limn/jit.py:109-135)
    and CudaDevice's buffer calls (limn/backend_cuda.py:316-350),
  * the frontend's call sequence: "sdpa" -> (O, L); delta = sum(dO * O); "sdpa_bwd_q" -> dQ
    and "sdpa_bwd_kv" -> (dK, dV) over (q, k, v, dO, L, delta[, mask]) (limn/tensor.py:559-574,
    :702-711), including the validation errors of Tensor.attention (limn/tensor.py:537-548).
It computes nothing itself; every value comes from the registered kernels.
"""

from __future__ import annotations

import math
from collections.abc import Callable, Sequence
from dataclasses import dataclass
from typing import Any

import ml_dtypes
import numpy as np

from limn_b200 import runtime
from limn_b200._lib import DTYPE_CODES, check, lib
from limn_b200.registry import SDPA, SDPA_BWD_KV, SDPA_BWD_Q, Runner, install


@dataclass(frozen=True)
class DType:
    name: str
    itemsize: int

    def __repr__(self) -> str:
        return self.name


float64 = DType("float64", 8)
float32 = DType("float32", 4)
float16 = DType("float16", 2)
bfloat16 = DType("bfloat16", 2)
FLOATS = (float64, float32, float16, bfloat16)
HALF_FLOATS = (float16, bfloat16)
NUMPY_DTYPES = {
    float64: np.dtype(np.float64),
    float32: np.dtype(np.float32),
    float16: np.dtype(np.float16),
    bfloat16: np.dtype(ml_dtypes.bfloat16),
}
FROM_NUMPY = {v: k for k, v in NUMPY_DTYPES.items()}


def accumulate_in(dtype: DType) -> DType:
    return float32 if dtype in HALF_FLOATS else dtype


@dataclass(frozen=True)
class Custom:
    name: str
    params: tuple
    outs: tuple[tuple[DType, tuple[int, ...]], ...]
    index: int = 0


@dataclass(eq=False)
class Node:
    srcs: tuple["Node", ...]
    dtype: DType
    shape: tuple[int, ...]
    arg: Any = None


def custom(name: str, srcs: tuple[Node, ...], params: tuple, outs: Sequence[tuple[DType, tuple[int, ...]]]) -> tuple[Node, ...]:
    specs = tuple(outs)
    return tuple(Node(srcs, dtype, shape, Custom(name, params, specs, index)) for index, (dtype, shape) in enumerate(specs))


class Device:
    """The slice of limn's CudaDevice the CUSTOM path uses, over limn_b200.runtime."""

    def __init__(self, ordinal: int = 0) -> None:
        runtime.set_device(ordinal)
        self.custom: dict[str, Callable[[Node], Runner]] = {}
        install(self)

    def has_custom(self, name: str) -> bool:
        return name in self.custom

    def custom_runner(self, node: Node) -> Runner:
        if (build := self.custom.get(node.arg.name)) is None:
            raise NotImplementedError(f"{type(self).__name__} has no kernel for custom op {node.arg.name!r}")
        return build(node)

    def prepare(self, array: np.ndarray) -> runtime.DeviceBuffer:
        return runtime.upload(array)

    def out_alloc(self, nbytes: int, zero: bool = False) -> runtime.DeviceBuffer:
        return runtime.empty(nbytes, poison=0 if zero else 0xFF)

    def copyout(self, buf: runtime.DeviceBuffer, dtype: DType, shape: tuple[int, ...]) -> np.ndarray:
        return runtime.download(buf, NUMPY_DTYPES[dtype], shape)

    def finish(self) -> None:
        runtime.synchronize()
        status = runtime.device_status()
        if status:
            raise RuntimeError(f"limn_b200: a kernel gave up on a bounded wait (status 0x{status:08x})")

    def call(self, nodes: tuple[Node, ...], inputs: list[runtime.DeviceBuffer]) -> list[runtime.DeviceBuffer]:
        """One merged call for a kernel's sibling nodes: a buffer per entry of `outs`, in
        output order, none zeroed (limn/jit.py:173-177, :215-224)."""
        runner = self.custom_runner(nodes[0])
        outs = [self.out_alloc(dtype.itemsize * math.prod(shape)) for dtype, shape in nodes[0].arg.outs]
        runner(inputs, outs)
        return outs


def _leaf(array: np.ndarray) -> Node:
    return Node((), FROM_NUMPY[array.dtype], tuple(array.shape))


def _validate(q: np.ndarray, k: np.ndarray, v: np.ndarray, key_mask, causal: bool) -> None:
    # limn/tensor.py:537-548
    if q.ndim < 2 or k.ndim < 2 or v.ndim < 2:
        raise ValueError(f"attention needs 2D+ tensors, got {q.shape}, {k.shape}, {v.shape}")
    if q.shape[-1] != k.shape[-1]:
        raise ValueError(f"attention: head dims differ, {q.shape[-1]} and {k.shape[-1]}")
    if k.shape[-2] != v.shape[-2]:
        raise ValueError(f"attention: key counts differ, {k.shape[-2]} and {v.shape[-2]}")
    if causal and q.shape[-2] != k.shape[-2]:
        raise ValueError(f"causal attention needs square keys, got {q.shape[-2]} queries and {k.shape[-2]} keys")
    if any(a.dtype not in FROM_NUMPY for a in (q, k, v)) or len({a.dtype for a in (q, k, v)}) != 1:
        raise ValueError(f"attention needs one float dtype, got {q.dtype}, {k.dtype}, {v.dtype}")
    if q.shape[:-2] != k.shape[:-2] or q.shape[:-2] != v.shape[:-2]:
        raise ValueError(f"attention: batch dims differ, {q.shape}, {k.shape}, {v.shape}")
    if key_mask is not None and key_mask.shape != q.shape[:-2] + k.shape[-2:-1]:
        raise ValueError(f"attention: a key mask ends in one flag per key, {k.shape[-2]}, got {key_mask.shape}")


class Attention:
    """One attention call held on the device: forward() then backward(dO), as autograd would."""

    def __init__(self, dev: Device, q: np.ndarray, k: np.ndarray, v: np.ndarray, *, causal: bool = False, key_mask=None):
        _validate(q, k, v, key_mask, causal)
        self.dev = dev
        self.causal = causal
        self.scale = q.shape[-1] ** -0.5
        self.dtype = FROM_NUMPY[q.dtype]
        self.shapes = (q.shape, k.shape, v.shape)
        mask = None if key_mask is None else np.ascontiguousarray(key_mask).astype(q.dtype)
        self.leaves = tuple(_leaf(a) for a in (q, k, v)) + (() if mask is None else (_leaf(mask),))
        self.bufs = [dev.prepare(a) for a in (q, k, v)] + ([] if mask is None else [dev.prepare(mask)])
        self.has_mask = mask is not None
        self.out_buf = self.lse_buf = None

    def forward(self) -> tuple[np.ndarray, np.ndarray]:
        (qs, ks, vs), wider = self.shapes, self.dtype
        batch = qs[:-2]
        outs = ((wider, batch + (qs[-2], vs[-1])), (accumulate_in(wider), batch + (qs[-2], 1)))
        self.fwd_nodes = custom(SDPA, self.leaves, (self.causal, self.scale), outs)
        self.out_buf, self.lse_buf = self.dev.call(self.fwd_nodes, self.bufs)
        self.dev.finish()
        return tuple(self.dev.copyout(buf, dtype, shape) for buf, (dtype, shape) in zip((self.out_buf, self.lse_buf), outs, strict=True))

    def backward(self, do: np.ndarray) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
        if self.out_buf is None:
            self.forward()
        (qs, ks, vs), wider = self.shapes, self.dtype
        saved = accumulate_in(wider)
        rows = math.prod(qs[:-1])
        do_buf = self.dev.prepare(np.ascontiguousarray(do).astype(NUMPY_DTYPES[wider]))
        delta_buf = self.dev.out_alloc(saved.itemsize * rows)
        check(
            lib().limn_b200_sdpa_delta(self.out_buf.ptr, do_buf.ptr, delta_buf.ptr, DTYPE_CODES[wider.name], rows, vs[-1], None),
            "launching the row dot",
        )
        q, k, v = self.leaves[:3]
        stat = (saved, qs[:-1] + (1,))
        held = (q, k, v, Node((), wider, qs[:-1] + vs[-1:]), Node((), *stat), Node((), *stat)) + self.leaves[3:]
        bufs = self.bufs[:3] + [do_buf, self.lse_buf, delta_buf] + self.bufs[3:]
        params = (self.causal, self.scale)
        dq_nodes = custom(SDPA_BWD_Q, held, params, ((wider, qs),))
        dkv_nodes = custom(SDPA_BWD_KV, held, params, ((wider, ks), (wider, vs)))
        (dq,) = self.dev.call(dq_nodes, bufs)
        dk, dv = self.dev.call(dkv_nodes, bufs)
        self.dev.finish()
        return (self.dev.copyout(dq, wider, qs), self.dev.copyout(dk, wider, ks), self.dev.copyout(dv, wider, vs))
