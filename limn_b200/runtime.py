"""Device memory for hosts that do not bring their own CUDA binding (the tests, the benchmark).

limn's cuda device allocates through the driver API and hands the kernels `CudaBuffer`
objects carrying `.ptr` and `.nbytes` (limn/backend_cuda.py:230-244). `DeviceBuffer` is the
same shape of object over the library's own plumbing calls, so a Runner built by
limn_b200.registry runs unchanged on either.
"""

from __future__ import annotations

import ctypes

import numpy as np

from limn_b200._lib import DEVICE_TIMEOUT, check, lib


class DeviceBuffer:
    """nbytes of device memory; freed when the last reference drops."""

    __slots__ = ("ptr", "nbytes")

    def __init__(self, nbytes: int):
        ptr = ctypes.c_void_p()
        check(lib().limn_b200_mem_alloc(ctypes.byref(ptr), nbytes), f"allocating {nbytes} bytes")
        self.ptr = ptr.value or 0
        self.nbytes = nbytes

    def __del__(self) -> None:
        try:
            if self.ptr:
                lib().limn_b200_mem_free(self.ptr)
                self.ptr = 0
        except Exception:  # interpreter teardown
            pass


def set_device(ordinal: int) -> None:
    check(lib().limn_b200_set_device(ordinal), f"selecting device {ordinal}")


def device_count() -> int:
    count = ctypes.c_int()
    check(lib().limn_b200_device_count(ctypes.byref(count)), "counting devices")
    return count.value


def upload(array: np.ndarray) -> DeviceBuffer:
    data = np.ascontiguousarray(array)
    buf = DeviceBuffer(data.nbytes)
    check(lib().limn_b200_copy_h2d(buf.ptr, data.ctypes.data, data.nbytes, None), "uploading bytes")
    check(lib().limn_b200_device_sync(), "waiting for an upload")
    return buf


def empty(nbytes: int, poison: int | None = 0xFF) -> DeviceBuffer:
    """Uninitialised output memory, as limn hands a kernel (limn/jit.py:173); filled with a
    poison byte so a kernel that leaves a gap shows it."""
    buf = DeviceBuffer(nbytes)
    if poison is not None and nbytes:
        check(lib().limn_b200_mem_set(buf.ptr, poison, nbytes, None), "poisoning an output")
    return buf


def download(buf: DeviceBuffer, dtype, shape) -> np.ndarray:
    check(lib().limn_b200_device_sync(), "waiting for the device")
    out = np.empty(buf.nbytes, dtype=np.uint8)
    check(lib().limn_b200_copy_d2h(out.ctypes.data, buf.ptr, buf.nbytes, None), "downloading bytes")
    check(lib().limn_b200_device_sync(), "waiting for a download")
    return out.view(dtype).reshape(shape)


def synchronize() -> None:
    check(lib().limn_b200_device_sync(), "waiting for the device")


def device_status() -> int:
    """The current device's kernel status word (0 = no kernel gave up on a wait); clears it."""
    word = ctypes.c_uint()
    code = lib().limn_b200_device_status(ctypes.byref(word))
    if code != DEVICE_TIMEOUT:  # a set word is this function's answer, not its failure
        check(code, "reading the device status word")
    return word.value


class Event:
    def __init__(self) -> None:
        handle = ctypes.c_void_p()
        check(lib().limn_b200_event_create(ctypes.byref(handle)), "creating an event")
        self.handle = handle.value

    def record(self, stream=None) -> None:
        handle = stream.handle if isinstance(stream, Stream) else stream
        check(lib().limn_b200_event_record(self.handle, handle), "recording an event")

    def ms_since(self, start: "Event") -> float:
        ms = ctypes.c_float()
        check(lib().limn_b200_event_elapsed_ms(start.handle, self.handle, ctypes.byref(ms)), "reading an event interval")
        return ms.value

    def __del__(self) -> None:
        try:
            lib().limn_b200_event_destroy(self.handle)
        except Exception:
            pass


class Stream:
    """A non-blocking CUDA stream (it does not synchronise with the legacy default stream)."""

    def __init__(self) -> None:
        handle = ctypes.c_void_p()
        check(lib().limn_b200_stream_create(ctypes.byref(handle)), "creating a stream")
        self.handle = handle.value

    def wait(self, event: Event) -> None:
        check(lib().limn_b200_stream_wait_event(self.handle, event.handle), "making a stream wait for an event")

    def synchronize(self) -> None:
        check(lib().limn_b200_stream_sync(self.handle), "waiting for a stream")

    def __del__(self) -> None:
        try:
            lib().limn_b200_stream_destroy(self.handle)
        except Exception:
            pass


class PinnedArray:
    """Page-locked host memory viewed as a numpy array: what asynchronous copies need at the host end."""

    def __init__(self, shape, dtype) -> None:
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(shape)) * self.dtype.itemsize
        ptr = ctypes.c_void_p()
        check(lib().limn_b200_host_alloc(ctypes.byref(ptr), self.nbytes), f"allocating {self.nbytes} pinned bytes")
        self.ptr = ptr.value
        raw = (ctypes.c_ubyte * self.nbytes).from_address(self.ptr)
        self.array = np.frombuffer(raw, dtype=np.uint8).view(self.dtype).reshape(shape)

    def __del__(self) -> None:
        try:
            if self.ptr:
                self.array = None
                lib().limn_b200_host_free(self.ptr)
                self.ptr = 0
        except Exception:
            pass
