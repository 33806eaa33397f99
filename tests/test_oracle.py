"""The CPU oracle held to the reference: golden vectors made by limn.sdpa itself, the
textbook softmax, span invariance and the edge cases the reference's own tests cover."""

from __future__ import annotations

import numpy as np
import pytest
from conftest import BF16, golden, widen

from oracle import sdpa_oracle as oracle

# worst() tolerance per storage dtype when both sides ran the same algorithm: fp32 differs by
# summation order only; a half-width output may land one rounding step apart.
TOL = {"float32": 2e-6, "float64": 1e-13, "float16": 1e-3, "bfloat16": 8e-3}
NAMES = golden().names()


@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_reference_golden(name, golden):
    q, k, v, do, mask, causal, scale = golden.inputs(name)
    tol = TOL[golden.cases[name][1]]
    out, lse = oracle.sdpa_forward(q, k, v, mask, causal=causal, scale=scale)
    want_out, want_lse = golden.output(name, "out"), golden.output(name, "lse")
    assert out.dtype == want_out.dtype and lse.dtype == want_lse.dtype and lse.shape == want_lse.shape
    assert oracle.worst(widen(out), widen(want_out)) <= tol
    assert oracle.worst(lse, want_lse) <= max(TOL["float32"], 1e-6) if lse.dtype == np.float32 else 1e-13
    # the backward ops are fed the reference's own O-derived statistics, so each op is pinned alone
    delta = golden.output(name, "delta")
    np.testing.assert_allclose(oracle.row_delta(do, want_out), delta, rtol=1e-5, atol=1e-5)
    dq = oracle.sdpa_backward_q(q, k, v, do, want_lse, delta, mask, causal=causal, scale=scale)
    dk, dv = oracle.sdpa_backward_kv(q, k, v, do, want_lse, delta, mask, causal=causal, scale=scale)
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        want = golden.output(name, key)
        assert got.dtype == want.dtype and got.shape == want.shape
        assert oracle.worst(widen(got), widen(want)) <= tol, key


def _textbook(q, k, v, do, mask, causal, scale):
    """Attention and its gradients with the whole t_q x t_k in memory, in float64."""
    Q, K, V, DO = (np.asarray(a).astype(np.float64) for a in (q, k, v, do))
    s = Q @ np.swapaxes(K, -1, -2) * scale
    if causal:
        t = s.shape[-1]
        s = np.where(np.tril(np.ones((t, t), bool)), s, -np.inf)
    if mask is not None:
        s = np.where((np.asarray(mask).astype(np.float64) != 0)[..., None, :], s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    dp = DO @ np.swapaxes(V, -1, -2)
    ds = p * (dp - (dp * p).sum(-1, keepdims=True)) * scale
    return p @ V, ds @ K, np.swapaxes(ds, -1, -2) @ Q, np.swapaxes(p, -1, -2) @ DO


@pytest.mark.parametrize("name", ["cfg1_f32_causal", "f32_rect_40x72", "f32_mask_holes", "f32_decode_row_mask", "f64_causal_hdv16"])
@pytest.mark.parametrize("span", [1, 16, 1000])
def test_oracle_equals_textbook_attention_at_any_span(name, span, golden):
    q, k, v, do, mask, causal, scale = golden.inputs(name)
    out, lse = oracle.sdpa_forward(q, k, v, mask, causal=causal, scale=scale, span=span)
    delta = oracle.row_delta(do, out)
    dq = oracle.sdpa_backward_q(q, k, v, do, lse, delta, mask, causal=causal, scale=scale, span=span)
    dk, dv = oracle.sdpa_backward_kv(q, k, v, do, lse, delta, mask, causal=causal, scale=scale, span=span)
    tol = 1e-12 if q.dtype == np.float64 else 1e-5
    for got, want in zip((out, dq, dk, dv), _textbook(q, k, v, do, mask, causal, scale), strict=True):
        assert oracle.worst(got, want) <= tol


def test_row_without_a_visible_key_is_nan_with_minus_inf_lse():
    rng = np.random.default_rng(1)
    q, k, v = (rng.standard_normal((2, 8, 4)).astype(np.float32) for _ in range(3))
    mask = np.ones((2, 8), np.float32)
    mask[1] = 0
    out, lse = oracle.sdpa_forward(q, k, v, mask, causal=False, scale=0.5)
    assert np.isfinite(out[0]).all() and np.isnan(out[1]).all()
    assert np.isneginf(lse[1]).all() and np.isfinite(lse[0]).all()


def test_hidden_keys_get_exactly_zero_gradients():
    rng = np.random.default_rng(2)
    q, k, v, do = (rng.standard_normal((3, 16, 8)).astype(np.float32) for _ in range(4))
    mask = (np.arange(16) < 11).astype(np.float32)[None].repeat(3, 0)
    out, lse = oracle.sdpa_forward(q, k, v, mask, causal=True, scale=8**-0.5)
    dk, dv = oracle.sdpa_backward_kv(q, k, v, do, lse, oracle.row_delta(do, out), mask, causal=True, scale=8**-0.5)
    assert (dk[:, 11:] == 0).all() and (dv[:, 11:] == 0).all() and np.abs(dk[:, :11]).min() > 0


def test_oracle_rejects_what_the_reference_rejects():
    z = np.zeros
    with pytest.raises(ValueError, match="square keys"):
        oracle.sdpa_forward(z((4, 8)), z((5, 8)), z((5, 8)), causal=True, scale=1.0)
    with pytest.raises(ValueError, match="head dims differ"):
        oracle.sdpa_forward(z((4, 8)), z((4, 6)), z((4, 8)), causal=False, scale=1.0)
    with pytest.raises(ValueError, match="shape mismatch"):
        oracle.sdpa_forward(z((2, 4, 8)), z((3, 4, 8)), z((3, 4, 8)), causal=False, scale=1.0)
    with pytest.raises(ValueError, match="key mask"):
        oracle.sdpa_forward(z((4, 8)), z((4, 8)), z((4, 8)), z((5,)), causal=False, scale=1.0)
    with pytest.raises(ValueError, match="equal rank"):
        oracle.sdpa_forward(z((8,)), z((8,)), z((8,)), causal=False, scale=1.0)


def test_half_width_inputs_round_once_at_the_end():
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((64, 32)).astype(BF16) for _ in range(3))
    out, lse = oracle.sdpa_forward(q, k, v, causal=True, scale=32**-0.5)
    wide, _ = oracle.sdpa_forward(*(a.astype(np.float32) for a in (q, k, v)), causal=True, scale=32**-0.5)
    assert out.dtype == BF16 and lse.dtype == np.float32
    np.testing.assert_array_equal(out, wide.astype(BF16))
