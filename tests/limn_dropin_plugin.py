"""pytest plugin that runs limn's own test-suite with limn_b200's kernels registered.

    cd <limn checkout> && python -m pytest -p limn_dropin_plugin tests/test_attention.py tests/test_jit.py

limn's tests build their cuda devices themselves (`backend_cuda.CudaDevice()` in their
conftest, `set_device("cuda")` inside tests), so the hook sits where every one of them
passes: CudaDevice.__init__ is wrapped to call limn_b200.install(self) once limn's own
constructor has filled the registry (limn/backend_cuda.py:292-293). Not one line of limn or of
its tests changes. The plugin loads before limn's conftest is imported (`-p` plugins load
first), so the shared `cudev` of that conftest is covered too.

It also counts how often each of the three builders and their Runners ran, and writes the
counts as JSON to the path in LIMN_B200_DROPIN_REPORT at the end of the session, so that a
caller can tell "limn's cuda attention tests passed on our kernels" from "they passed on
limn's NVRTC kernels because nothing was installed".
"""

from __future__ import annotations

import json
import os

import limn_b200
from limn_b200 import registry

COUNTS = {name: {"built": 0, "ran": 0} for name in registry.NAMES}


def _counting(name, build):
    def counted_build(node):
        COUNTS[name]["built"] += 1
        run = build(node)

        def counted_run(inputs, outs):
            COUNTS[name]["ran"] += 1
            run(inputs, outs)

        return counted_run

    return counted_build


def _patch() -> None:
    from limn import backend_cuda

    original = backend_cuda.CudaDevice.__init__
    if getattr(original, "_limn_b200_patched", False):
        return

    def __init__(self, *args, **kwargs):
        original(self, *args, **kwargs)
        limn_b200.install(self)
        for name in registry.NAMES:
            self.custom[name] = _counting(name, self.custom[name])

    __init__._limn_b200_patched = True
    backend_cuda.CudaDevice.__init__ = __init__


_patch()


def pytest_sessionfinish(session, exitstatus):
    path = os.environ.get("LIMN_B200_DROPIN_REPORT")
    if path:
        with open(path, "w") as handle:
            json.dump({"exitstatus": int(exitstatus), "counts": COUNTS}, handle)
