"""CPU oracle for the fused-attention CUSTOM ops (test infrastructure, not product code).

This is a numpy restatement of the algorithm limn's numpy device runs for the three CUSTOM
names "sdpa", "sdpa_bwd_q" and "sdpa_bwd_kv" (limn/sdpa.py:91-203, dispatched from
limn/device.py:160-167 through the registry at limn/sdpa.py:209-221). Only tests, the
smoke check and the benchmark's CPU-baseline leg may import it; the library itself never
does, and has no CPU path at all.

Parity is pinned: tests/golden/ holds input/output vectors produced by importing the
reference's own limn.sdpa functions (tests/golden/make_golden.py is the generator), and
tests/test_oracle.py holds this file to them.

Conventions, all taken from the reference:
  * q is (..., t_q, hd), k is (..., t_k, hd), v is (..., t_k, hd_v); leading dims equal.
  * half-width storage (float16, bfloat16) is widened to float32 for the whole recurrence
    and rounded once at the end (limn/sdpa.py:48-51, :137, :170, :203); float32 and float64
    run at their own width.
  * causal keeps key j for query i when j <= i and needs t_q == t_k (limn/sdpa.py:65-66,
    :86-87); key_mask is (..., t_k), 0 hides the key from every query (limn/sdpa.py:70-74, :88).
  * a hidden score contributes exactly 0; a query with no visible key returns NaN and an
    L of -inf (limn/sdpa.py:111-112, :126-129).
  * L = running_max + log(running_sum), shaped (..., t_q, 1), at the working width
    (limn/sdpa.py:136).
  * delta = sum_d dO * O over the *rounded* O, at the working width (limn/tensor.py:705-706).
"""

from __future__ import annotations

import ml_dtypes
import numpy as np

BF16 = np.dtype(ml_dtypes.bfloat16)
NARROW = (np.dtype(np.float16), BF16)

# How many keys (or queries) one step of the recurrence folds in. The reference's registry
# entry runs its default of 16 (limn/sdpa.py:99); the result does not depend on it beyond
# rounding, which tests/test_oracle.py checks by sweeping it.
DEFAULT_SPAN = 16


def working_dtype(dtype) -> np.dtype:
    """float32 for the two half-width storage types, the type itself otherwise."""
    dtype = np.dtype(dtype)
    return np.dtype(np.float32) if dtype in NARROW else dtype


def _check_shapes(q, k, v, key_mask, causal) -> None:
    # limn/sdpa.py:58-74
    if q.ndim < 2 or k.ndim != q.ndim or v.ndim != q.ndim:
        raise ValueError(f"sdpa wants 2D+ inputs of equal rank, got {q.shape}, {k.shape}, {v.shape}")
    lead = q.shape[:-2]
    if k.shape[:-2] != lead or v.shape[:-2] != lead or k.shape[-2] != v.shape[-2]:
        raise ValueError(f"sdpa shape mismatch: {q.shape}, {k.shape}, {v.shape}")
    if q.shape[-1] != k.shape[-1]:
        raise ValueError(f"sdpa: head dims differ, {q.shape[-1]} and {k.shape[-1]}")
    if causal and q.shape[-2] != k.shape[-2]:
        raise ValueError(f"causal sdpa needs square keys, got {q.shape[-2]} queries and {k.shape[-2]} keys")
    if key_mask is not None and key_mask.shape != lead + (k.shape[-2],):
        raise ValueError(f"sdpa key mask must be {lead + (k.shape[-2],)}, got {key_mask.shape}")


def _visible(t_q: int, i0: int, i1: int, j0: int, j1: int, causal: bool, key_mask) -> np.ndarray | None:
    """Boolean (…, i1-i0, j1-j0) of which (query, key) pairs of a tile take part, or None for all."""
    keep = None
    if causal:
        keep = np.arange(j0, j1)[None, :] <= np.arange(i0, i1)[:, None]
    if key_mask is not None:
        live = (key_mask[..., j0:j1] != 0)[..., None, :]
        keep = live if keep is None else np.logical_and(keep, live)
    return keep


def _tile_scores(Q, K, i0, i1, j0, j1, causal, scale, key_mask) -> np.ndarray:
    """scale * Q[i0:i1] K[j0:j1]^T with hidden pairs at -inf (limn/sdpa.py:77-88)."""
    s = np.matmul(Q[..., i0:i1, :], np.swapaxes(K[..., j0:j1, :], -1, -2)) * Q.dtype.type(scale)
    keep = _visible(Q.shape[-2], i0, i1, j0, j1, causal, key_mask)
    if keep is not None:
        s = np.where(keep, s, Q.dtype.type(-np.inf))
    return s


def sdpa_forward(q, k, v, key_mask=None, *, causal: bool, scale: float, span: int = DEFAULT_SPAN):
    """O = softmax(scale * q k^T, hidden pairs removed) v and L = logsumexp per query row.

    Online softmax over spans of keys, as limn/sdpa.py:114-137: a running max m, a running
    denominator l and a running numerator per row; raising m to m' multiplies what was
    accumulated by exp(m - m'). Returns (O in q's dtype, L in the working dtype, shape (..., t_q, 1)).
    """
    _check_shapes(q, k, v, key_mask, causal)
    work = working_dtype(q.dtype)
    Q, K, V = (np.asarray(a).astype(work, copy=False) for a in (q, k, v))
    t_q, t_k = q.shape[-2], k.shape[-2]
    lead = q.shape[:-2]
    numer = np.zeros(lead + (t_q, v.shape[-1]), dtype=work)
    denom = np.zeros(lead + (t_q,), dtype=work)
    top = np.full(lead + (t_q,), -np.inf, dtype=work)
    for j0 in range(0, t_k, span):
        j1 = min(j0 + span, t_k)
        s = _tile_scores(Q, K, 0, t_q, j0, j1, causal, scale, key_mask)
        raised = np.maximum(top, s.max(axis=-1))
        # a row that has met no visible key yet has raised == -inf; subtracting that from
        # itself would be NaN, so such a row is measured against 0 and both of its factors
        # come out exp(-inf) = 0 (limn/sdpa.py:126-129)
        base = np.where(np.isneginf(raised), work.type(0), raised)
        shrink = np.exp(top - base)
        w = np.exp(s - base[..., None])
        denom = denom * shrink + w.sum(axis=-1)
        numer = numer * shrink[..., None] + np.matmul(w, V[..., j0:j1, :])
        top = raised
    with np.errstate(divide="ignore", invalid="ignore"):
        lse = (top + np.log(denom))[..., None]
        out = (numer / denom[..., None]).astype(q.dtype)
    return out, lse


def row_delta(do, out) -> np.ndarray:
    """delta_i = sum_d dO_id * O_id at the working width, shape (..., t_q, 1) (limn/tensor.py:705-706)."""
    work = working_dtype(out.dtype)
    return (np.asarray(do).astype(work) * np.asarray(out).astype(work)).sum(axis=-1, keepdims=True)


def _widen_all(*arrays):
    work = working_dtype(arrays[0].dtype)
    return [np.asarray(a).astype(work, copy=False) for a in arrays]


def sdpa_backward_q(q, k, v, do, lse, delta, key_mask=None, *, causal: bool, scale: float, span: int = DEFAULT_SPAN):
    """dQ_i = sum_j p_ij (dP_ij - delta_i) scale K_j, p_ij = exp(scale s_ij - L_i), dP_ij = dO_i . V_j.

    Keys are folded in spans; nothing t_q-by-t_k is kept (limn/sdpa.py:140-170).
    """
    _check_shapes(q, k, v, key_mask, causal)
    Q, K, V, DO, L, DL = _widen_all(q, k, v, do, lse, delta)
    t_q, t_k = q.shape[-2], k.shape[-2]
    dq = np.zeros_like(Q)
    for j0 in range(0, t_k, span):
        j1 = min(j0 + span, t_k)
        s = _tile_scores(Q, K, 0, t_q, j0, j1, causal, scale, key_mask)
        p = np.exp(s - L)  # a hidden pair is exp(-inf) = 0 exactly
        dp = np.matmul(DO, np.swapaxes(V[..., j0:j1, :], -1, -2))
        ds = p * (dp - DL) * Q.dtype.type(scale)
        dq += np.matmul(ds, K[..., j0:j1, :])
    return dq.astype(q.dtype)


def sdpa_backward_kv(q, k, v, do, lse, delta, key_mask=None, *, causal: bool, scale: float, span: int = DEFAULT_SPAN):
    """dV_j = sum_i p_ij dO_i and dK_j = sum_i ds_ij Q_i with the same p and ds as sdpa_backward_q.

    Queries are folded in spans against all keys (limn/sdpa.py:173-203). A hidden key has
    p = 0 for every query, so its dK and dV rows are exactly zero.
    """
    _check_shapes(q, k, v, key_mask, causal)
    Q, K, V, DO, L, DL = _widen_all(q, k, v, do, lse, delta)
    t_q, t_k = q.shape[-2], k.shape[-2]
    dk = np.zeros_like(K)
    dv = np.zeros_like(V)
    for i0 in range(0, t_q, span):
        i1 = min(i0 + span, t_q)
        s = _tile_scores(Q, K, i0, i1, 0, t_k, causal, scale, key_mask)
        p = np.exp(s - L[..., i0:i1, :])
        dv += np.matmul(np.swapaxes(p, -1, -2), DO[..., i0:i1, :])
        dp = np.matmul(DO[..., i0:i1, :], np.swapaxes(V, -1, -2))
        ds = p * (dp - DL[..., i0:i1, :]) * Q.dtype.type(scale)
        dk += np.matmul(np.swapaxes(ds, -1, -2), Q[..., i0:i1, :])
    return dk.astype(k.dtype), dv.astype(v.dtype)


def run_custom(name: str, srcs, causal: bool, scale: float):
    """The registry view of the three ops: (name, inputs in node order, params) -> tuple of outputs.

    Input order follows the CUSTOM nodes the frontend builds (limn/tensor.py:563-567 for the
    forward, :707-711 for the two backward ops); an optional key mask rides last.
    """
    if name == "sdpa":
        return sdpa_forward(*srcs, causal=causal, scale=scale)
    if name == "sdpa_bwd_q":
        return (sdpa_backward_q(*srcs, causal=causal, scale=scale),)
    if name == "sdpa_bwd_kv":
        return sdpa_backward_kv(*srcs, causal=causal, scale=scale)
    raise KeyError(name)


def worst(got: np.ndarray, want: np.ndarray) -> float:
    """max |got - want| relative to max(1, max |want|): the reference checker's error measure
    (limn/sdpa.py:251-259)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(got - want).max() / max(1.0, float(np.abs(want).max())))
