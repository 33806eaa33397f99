"""The drop-in point: builders for limn's CUSTOM registry on a cuda device.

limn's plan executor asks `device.custom[name](node)` for a `Runner` once per plan and then
calls `runner(inputs, outs)` every step (limn/jit.py:41, :109, :130-135, :213-224). The
reference's CudaDevice fills the registry with a builder that emits CUDA C and compiles it
with NVRTC (limn/backend_cuda.py:292-293, :352-361). `install(dev)` overwrites the three
entries with builders that bind the prebuilt sm_100a kernels instead; nothing else in limn
changes, and tensor.py's `has_custom` checks (limn/tensor.py:559, :696) keep passing.

A builder reads only what the node states: `node.arg.name`, `node.arg.params == (causal,
scale)`, `node.arg.outs`, and each `node.srcs[i].shape` / `.dtype.name`; so it works on
limn's Node or on a test's stand-in alike. A Runner reads `.ptr` off every buffer
on every call and keeps none of them, because a captured plan is replayed against new
buffers each time (limn/capture.py:152-168). It launches on the legacy default stream, where
limn's own kernels run (limn/backend_cuda.py:413), and does not synchronise: the device's
finish() does that once per batch (limn/jit.py:183).
"""

from __future__ import annotations

import math
from collections.abc import Callable
from typing import Any

import ctypes

from limn_b200._lib import DEVICE_TIMEOUT, DTYPE_CODES, check, lib

SDPA, SDPA_BWD_Q, SDPA_BWD_KV = "sdpa", "sdpa_bwd_q", "sdpa_bwd_kv"  # limn/sdpa.py:43-45
NAMES = (SDPA, SDPA_BWD_Q, SDPA_BWD_KV)

Runner = Callable[[list[Any], list[Any]], None]


class Form:
    """A CUSTOM attention node read as extents: what limn/cuda_emit.py:890-918 reads off the
    same node. `inputs` is the op's input count without a key mask; one more means the last
    one is the mask."""

    def __init__(self, node: Any, inputs: int):
        causal, scale = node.arg.params
        q, k, v = node.srcs[:3]
        if q.dtype.name not in DTYPE_CODES:
            raise NotImplementedError(f"limn_b200: {node.arg.name} has no kernel for dtype {q.dtype.name}")
        for src in (k, v):
            if src.dtype.name != q.dtype.name:
                raise ValueError(f"limn_b200: {node.arg.name} wants one dtype, got {q.dtype.name} and {src.dtype.name}")
        if len(q.shape) < 2 or len(k.shape) != len(q.shape) or len(v.shape) != len(q.shape):
            raise ValueError(f"limn_b200: {node.arg.name} wants 2D+ inputs of equal rank, got {q.shape}, {k.shape}, {v.shape}")
        if q.shape[:-2] != k.shape[:-2] or q.shape[:-2] != v.shape[:-2] or k.shape[-2] != v.shape[-2]:
            raise ValueError(f"limn_b200: {node.arg.name} shape mismatch: {q.shape}, {k.shape}, {v.shape}")
        if q.shape[-1] != k.shape[-1]:
            raise ValueError(f"limn_b200: {node.arg.name}: head dims differ, {q.shape[-1]} and {k.shape[-1]}")
        if causal and q.shape[-2] != k.shape[-2]:
            raise ValueError(
                f"limn_b200: causal {node.arg.name} needs square keys, got {q.shape[-2]} queries and {k.shape[-2]} keys"
            )
        if len(node.srcs) not in (inputs, inputs + 1):
            raise ValueError(f"limn_b200: {node.arg.name} takes {inputs} inputs and an optional key mask, got {len(node.srcs)}")
        self.name = node.arg.name
        self.causal = bool(causal)
        self.scale = float(scale)
        self.dtype = DTYPE_CODES[q.dtype.name]
        self.bh = math.prod(q.shape[:-2])
        self.t_q, self.t_k = q.shape[-2], k.shape[-2]
        self.hd, self.hd_v = q.shape[-1], v.shape[-1]
        self.has_mask = len(node.srcs) > inputs
        self.inputs = len(node.srcs)
        self.outputs = len(node.arg.outs)

    def tail(self) -> tuple:
        return (self.dtype, self.bh, self.t_q, self.t_k, self.hd, self.hd_v, int(self.causal), self.scale, None)


def _pointers(form: Form, inputs: list[Any], outs: list[Any]) -> tuple[list[int], list[int]]:
    if len(inputs) != form.inputs or len(outs) != form.outputs:
        raise RuntimeError(
            f"limn_b200: {form.name} was built for {form.inputs} inputs and {form.outputs} outputs, "
            f"called with {len(inputs)} and {len(outs)}"
        )
    return [buf.ptr for buf in inputs], [buf.ptr for buf in outs]


def build_sdpa(node: Any) -> Runner:
    """Runner for "sdpa": inputs (q, k, v[, mask]) -> outs (O, L). Stands where
    CudaDevice._sdpa_runner stands for this name (limn/backend_cuda.py:352-361)."""
    form = Form(node, 3)
    fn = lib().limn_b200_sdpa_fwd
    tail = form.tail()

    def run(inputs: list[Any], outs: list[Any]) -> None:
        ins, (out, lse) = _pointers(form, inputs, outs)
        mask = ins[3] if form.has_mask else None
        check(fn(ins[0], ins[1], ins[2], mask, out, lse, *tail), "launching sdpa")
        _note_launch()

    return run


def build_sdpa_bwd_q(node: Any) -> Runner:
    """Runner for "sdpa_bwd_q": inputs (q, k, v, dO, L, delta[, mask]) -> outs (dQ,)."""
    form = Form(node, 6)
    fn = lib().limn_b200_sdpa_bwd_q
    tail = form.tail()

    def run(inputs: list[Any], outs: list[Any]) -> None:
        ins, (dq,) = _pointers(form, inputs, outs)
        mask = ins[6] if form.has_mask else None
        check(fn(ins[0], ins[1], ins[2], ins[3], ins[4], ins[5], mask, dq, *tail), "launching sdpa_bwd_q")
        _note_launch()

    return run


def build_sdpa_bwd_kv(node: Any) -> Runner:
    """Runner for "sdpa_bwd_kv": inputs (q, k, v, dO, L, delta[, mask]) -> outs (dK, dV)."""
    form = Form(node, 6)
    fn = lib().limn_b200_sdpa_bwd_kv
    tail = form.tail()

    def run(inputs: list[Any], outs: list[Any]) -> None:
        ins, (dk, dv) = _pointers(form, inputs, outs)
        mask = ins[6] if form.has_mask else None
        check(fn(ins[0], ins[1], ins[2], ins[3], ins[4], ins[5], mask, dk, dv, *tail), "launching sdpa_bwd_kv")
        _note_launch()

    return run


def build_sdpa_bwd_q_fused(node: Any) -> Runner:
    """Runner for "sdpa_bwd_q_fused": inputs (q, k, v, O, dO, L[, mask]) -> outs (dQ, delta). Not one of limn's
    names: the node only exists once limn_b200.frontend.fuse_row_dot() has taught the frontend to build it in
    place of its row-dot reduce followed by "sdpa_bwd_q" (limn/tensor.py:702-710)."""
    form = Form(node, 6)
    fn = lib().limn_b200_sdpa_bwd_q_fused
    tail = form.tail()

    def run(inputs: list[Any], outs: list[Any]) -> None:
        ins, (dq, delta) = _pointers(form, inputs, outs)
        mask = ins[6] if form.has_mask else None
        check(fn(ins[0], ins[1], ins[2], ins[3], ins[4], ins[5], mask, dq, delta, *tail), "launching sdpa_bwd_q_fused")
        _note_launch()

    return run


class StridedForm:
    """A "*_strided" CUSTOM node (built by limn_b200.frontend.read_views_in_place): srcs are the buffers under the
    operands' views, params carry (causal, scale, (batch, heads, t_q, t_k, hd), per-view (offset, batch, head, row
    strides) in elements). Several operands may sit on one buffer (q, k and v of one projection): the plan then
    hands that buffer over once (limn/schedule.py: fuse() lists a kernel's inputs without repeats), in the order
    of first appearance among the srcs, which `slot` reproduces."""

    def __init__(self, node: Any, outputs: int):
        self.name = node.arg.name
        causal, scale, (batch, heads, t_q, t_k, hd), self.views = node.arg.params
        self.causal, self.scale = bool(causal), float(scale)
        self.batch, self.heads, self.t_q, self.t_k, self.hd = batch, heads, t_q, t_k, hd
        dtype = node.srcs[0].dtype
        if dtype.name not in ("float16", "bfloat16"):
            raise NotImplementedError(f"limn_b200: {self.name} has no kernel for dtype {dtype.name}")
        self.dtype = DTYPE_CODES[dtype.name]
        unique = list(dict.fromkeys(node.srcs))
        self.slot = [unique.index(src) for src in node.srcs]
        self.inputs = len(unique)
        if len(node.arg.outs) != outputs:
            raise ValueError(f"limn_b200: {self.name} writes {outputs} outputs, the node declares {len(node.arg.outs)}")
        self.outputs = outputs

    def token_major(self, t: int) -> tuple[int, int, int]:
        """(batch, head, row) strides of a dense (batch, t, heads, hd) result."""
        return (t * self.heads * self.hd, self.hd, self.heads * self.hd)

    def strides(self, *triples: tuple[int, int, int]):
        flat = [x for triple in triples for x in triple]
        return (ctypes.c_longlong * len(flat))(*flat)

    def tail(self) -> tuple:
        return (self.dtype, self.batch, self.heads, self.t_q, self.t_k, self.hd, self.hd, int(self.causal), self.scale, None)

    def pointers(self, inputs: list[Any], outs: list[Any]) -> tuple[list[int], list[int]]:
        if len(inputs) != self.inputs or len(outs) != self.outputs:
            raise RuntimeError(
                f"limn_b200: {self.name} was built for {self.inputs} buffers and {self.outputs} outputs, "
                f"called with {len(inputs)} and {len(outs)}"
            )
        return [inputs[s].ptr for s in self.slot], [buf.ptr for buf in outs]


def build_sdpa_strided(node: Any) -> Runner:
    """Runner for "sdpa_strided": buffers under (q, k, v) -> outs (O token-major, L)."""
    form = StridedForm(node, 2)
    fn = lib().limn_b200_sdpa_fwd_strided
    strides = form.strides(*[view[1:] for view in form.views[:3]], form.token_major(form.t_q))
    offsets = [view[0] * 2 for view in form.views[:3]]
    tail = form.tail()

    def run(inputs: list[Any], outs: list[Any]) -> None:
        ins, (out, lse) = form.pointers(inputs, outs)
        q, k, v = (ins[i] + offsets[i] for i in range(3))
        check(fn(q, k, v, None, out, lse, strides, *tail), "launching sdpa_strided")
        _note_launch()

    return run


def build_sdpa_bwd_q_fused_strided(node: Any) -> Runner:
    """Runner for "sdpa_bwd_q_fused_strided": buffers under (q, k, v), O, buffer under dO, L -> outs (dQ token-major, delta)."""
    form = StridedForm(node, 2)
    fn = lib().limn_b200_sdpa_bwd_q_fused_strided
    major = form.token_major(form.t_q)
    strides = form.strides(*[view[1:] for view in form.views[:3]], major, form.views[3][1:], major)
    offsets = [view[0] * 2 for view in form.views]
    tail = form.tail()

    def run(inputs: list[Any], outs: list[Any]) -> None:
        ins, (dq, delta) = form.pointers(inputs, outs)
        q, k, v = (ins[i] + offsets[i] for i in range(3))
        check(fn(q, k, v, ins[3], ins[4] + offsets[3], ins[5], None, dq, delta, strides, *tail), "launching sdpa_bwd_q_fused_strided")
        _note_launch()

    return run


def build_sdpa_bwd_kv_strided(node: Any) -> Runner:
    """Runner for "sdpa_bwd_kv_strided": buffers under (q, k, v), buffer under dO, L, delta -> outs (dK, dV token-major)."""
    form = StridedForm(node, 2)
    fn = lib().limn_b200_sdpa_bwd_kv_strided
    major = form.token_major(form.t_k)
    strides = form.strides(*[view[1:] for view in form.views[:3]], form.views[3][1:], major, major)
    offsets = [view[0] * 2 for view in form.views]
    tail = form.tail()

    def run(inputs: list[Any], outs: list[Any]) -> None:
        ins, (dk, dv) = form.pointers(inputs, outs)
        q, k, v = (ins[i] + offsets[i] for i in range(3))
        check(fn(q, k, v, ins[3] + offsets[3], ins[4], ins[5], None, dk, dv, strides, *tail), "launching sdpa_bwd_kv_strided")
        _note_launch()

    return run


SDPA_BWD_Q_FUSED = "sdpa_bwd_q_fused"
BUILDERS: dict[str, Callable[[Any], Runner]] = {
    SDPA: build_sdpa,
    SDPA_BWD_Q: build_sdpa_bwd_q,
    SDPA_BWD_KV: build_sdpa_bwd_kv,
    SDPA_BWD_Q_FUSED: build_sdpa_bwd_q_fused,
    "sdpa_strided": build_sdpa_strided,
    "sdpa_bwd_q_fused_strided": build_sdpa_bwd_q_fused_strided,
    "sdpa_bwd_kv_strided": build_sdpa_bwd_kv_strided,
}


# Whether a Runner has launched since the last status check: finish() only pays for the check then.
_launched_since_check = False


def _note_launch() -> None:
    global _launched_since_check
    _launched_since_check = True


def check_device_status(doing: str = "waiting for the batch") -> None:
    """Raise if a kernel of this library gave up on a bounded wait since the last check.

    A kernel that waits (on a TMA copy or on the tensor pipe) does so for a bounded time; when
    the time runs out it records a code in a per-device status word and returns, and every
    later kernel on that device returns at once without writing its outputs until the word has
    been read. The reference turns a failed kernel into a RuntimeError at its batch barrier
    (limn/backend_cuda.py:349 through check(), :154-162); this is the same for ours."""
    global _launched_since_check
    if not _launched_since_check:
        return
    _launched_since_check = False
    word = ctypes.c_uint(0)
    code = lib().limn_b200_device_status(ctypes.byref(word))
    if code != DEVICE_TIMEOUT:
        check(code, "reading the device status word")
    if word.value:
        raise RuntimeError(
            f"cuda: {doing}: a limn_b200 kernel gave up on a bounded wait (status 0x{word.value:08x}); "
            "outputs of this batch are incomplete"
        )


def install(device: Any) -> Any:
    """Register the builders on a device that has a `custom` registry (limn's CompiledDevice,
    limn/jit.py:103-135): limn's three names, and the names limn's frontend only asks for once it has been
    patched: "sdpa_bwd_q_fused" (limn_b200.frontend.fuse_row_dot) and the three "*_strided" ones
    (limn_b200.frontend.read_views_in_place). Loads the shared library first, so a missing or
    unloadable library fails here rather than at the first step.

    The device's finish() (limn's one synchronise per batch, limn/jit.py:183) is wrapped so that
    after it returns the kernels' status word is read whenever one of our Runners ran in the
    batch: a kernel that gave up surfaces as a RuntimeError at the same place a failed kernel of
    the reference's does, instead of as unwritten buffers later."""
    lib()
    if not hasattr(device, "custom"):
        raise TypeError(f"limn_b200.install: {type(device).__name__} has no CUSTOM registry")
    for name, build in BUILDERS.items():
        device.custom[name] = build
    inner = getattr(device, "finish", None)
    if callable(inner) and not getattr(inner, "_limn_b200_checked", False):

        def finish() -> None:
            inner()
            check_device_status()

        finish._limn_b200_checked = True  # type: ignore[attr-defined]
        device.finish = finish
    return device
