"""Shared fixtures: the `gpu` marker, the golden bundle and a loader for its cases."""

from __future__ import annotations

import sys
from pathlib import Path

import ml_dtypes
import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
for extra in (ROOT, ROOT / "tests" / "golden"):
    if str(extra) not in sys.path:
        sys.path.insert(0, str(extra))

BF16 = np.dtype(ml_dtypes.bfloat16)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


class Golden:
    """tests/golden/sdpa_golden.npz: outputs of the reference's numpy kernels on seeded inputs.

    Inputs are regenerated from the seeds by the same function the generator used."""

    def __init__(self) -> None:
        import make_golden

        self.cases = {case[0]: case for case in make_golden.CASES}
        self.inputs_for = make_golden.inputs_for
        self.bundle = np.load(ROOT / "tests" / "golden" / "sdpa_golden.npz")

    def names(self) -> list[str]:
        return list(self.cases)

    def inputs(self, name: str):
        return self.inputs_for(self.cases[name])

    def output(self, name: str, key: str) -> np.ndarray:
        full = f"{name}/{key}"
        if full + "__bf16" in self.bundle:
            return self.bundle[full + "__bf16"].view(BF16)
        return self.bundle[full]


_golden: Golden | None = None


def golden() -> Golden:
    global _golden
    if _golden is None:
        _golden = Golden()
    return _golden


@pytest.fixture(scope="session", name="golden")
def golden_fixture() -> Golden:
    return golden()


def widen(a: np.ndarray) -> np.ndarray:
    """Half-width results are compared as float32, as the reference's own check does (tests/conftest.py:67-68)."""
    return a.astype(np.float32) if a.dtype in (np.dtype(np.float16), BF16) else a
