"""Shared fixtures: the `gpu` marker, the golden bundle and a loader for its cases, and the one
parity gate every comparison with the oracle goes through (it records both error measures)."""

from __future__ import annotations

import json
import os
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


# ---- the parity gate ----
# Two measures of the same difference: the raw max-abs error, which is what the path's tolerances are stated in
# (2e-2 for bfloat16 inputs, 1e-4 for float32, 1e-3 for the log-sum-exp), and the reference checker's measure,
# max-abs / max(1, max |want|) (limn/sdpa.py:251-259). Where the answer stays within [-1, 1] they are the same
# number and the gate is the raw one. Where it does not (gradients under a sharp softmax reach tens), one
# bfloat16 step of the answer alone exceeds 2e-2, so the gate is the normalised figure there. Every call is
# recorded with both, and the session leaves the table behind if LIMN_B200_TEST_REPORTS names a directory.
PARITY_ROWS: list[dict] = []


def parity(got: np.ndarray, want: np.ndarray, tol: float, what: str) -> tuple[float, float]:
    """Assert got ~ want under the rule above; returns (raw max-abs, normalised error)."""
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    g, w = widen(got).astype(np.float64), widen(want).astype(np.float64)
    finite = np.isfinite(w)
    assert np.array_equal(np.isnan(g), np.isnan(w)), f"{what}: NaNs are not where the oracle has them"
    assert np.array_equal(g[~finite & ~np.isnan(w)], w[~finite & ~np.isnan(w)]), f"{what}: infinities differ"
    raw = float(np.abs(g[finite] - w[finite]).max()) if finite.any() else 0.0
    biggest = float(np.abs(w[finite]).max()) if finite.any() else 0.0
    normalised = raw / max(1.0, biggest)
    gated_on = "raw" if biggest <= 1.0 else "normalised"
    PARITY_ROWS.append({"what": what, "max_abs_want": biggest, "raw": raw, "normalised": normalised, "tol": tol, "gate": gated_on})
    assert normalised <= tol, f"{what}: {gated_on} error {normalised:.3e} > {tol:g} (raw max-abs {raw:.3e}, max |want| {biggest:.3g})"
    return raw, normalised


def pytest_sessionfinish(session, exitstatus):
    keep = os.environ.get("LIMN_B200_TEST_REPORTS")
    if keep and PARITY_ROWS and os.path.isdir(keep):
        with open(os.path.join(keep, "parity_rows.json"), "w") as handle:
            json.dump(PARITY_ROWS, handle)
