"""Parity of the CUDA kernels, called through the C ABI and the registry builders, against
the reference-made golden vectors and the CPU oracle. Shaped after the reference's own
cuda-vs-numpy tests (tests/test_attention.py:243-396 there)."""

from __future__ import annotations

import numpy as np
import pytest
from conftest import BF16, golden, parity, widen

from oracle import sdpa_oracle as oracle

pytestmark = pytest.mark.gpu

# Tolerances: 1e-4 for fp32 inputs, 2e-2 for bf16 inputs, 1e-3 for the log-sum-exp; fp16 and fp64 take the
# reference's own cuda-vs-numpy tolerances (tests/test_attention.py:250-255, :303-308 and limn/sdpa.py:285).
# They gate the raw max-abs error wherever the answer stays within [-1, 1] and the error relative to the
# answer's largest magnitude elsewhere (conftest.parity, which records both figures for every comparison).
FWD_TOL = {"float32": 1e-4, "bfloat16": 2e-2, "float16": 2e-3, "float64": 1e-11}
BWD_TOL = {"float32": 1e-4, "bfloat16": 2e-2, "float16": 4e-3, "float64": 1e-11}
LSE_TOL = 1e-3


@pytest.fixture(scope="module")
def dev():
    import limn_standin as host

    return host.Device()


def close(got, want, tol, what) -> None:
    """The shared gate (conftest.parity): raw max-abs <= tol where the answer stays within [-1, 1], relative to
    the answer's size where it is larger (the reference's own measure, limn/sdpa.py:251-259); both recorded."""
    assert got.dtype == want.dtype, what
    parity(got, want, tol, what)


@pytest.mark.parametrize("name", golden().names())
def test_kernels_match_reference_golden(name, dev, golden):
    import limn_standin as host

    q, k, v, do, mask, causal, scale = golden.inputs(name)
    dtype = golden.cases[name][1]
    att = host.Attention(dev, q, k, v, causal=causal, key_mask=mask)
    out, lse = att.forward()
    close(out, golden.output(name, "out"), FWD_TOL[dtype], f"{name} O")
    close(lse, golden.output(name, "lse"), LSE_TOL if dtype != "float64" else 1e-11, f"{name} L")
    dq, dk, dv = att.backward(do)
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        close(got, golden.output(name, key), BWD_TOL[dtype], f"{name} {key}")


def _random_case(seed, dtype, qs, ks, vs, q_mul=1.0, v_uniform=False):
    rng = np.random.default_rng(seed)
    q = (rng.standard_normal(qs) * q_mul).astype(dtype)
    k = (rng.standard_normal(ks) * q_mul).astype(dtype)
    v = (rng.uniform(-1, 1, vs) if v_uniform else rng.standard_normal(vs)).astype(dtype)
    do = rng.standard_normal(qs[:-1] + vs[-1:]).astype(dtype)
    return q, k, v, do


ORACLE_CASES = [
    # id, dtype, q, k, v shapes, causal, q/k multiplier, uniform V
    ("bf16 d128 causal 5 tiles", BF16, (2, 3, 640, 128), (2, 3, 640, 128), (2, 3, 640, 128), True, 0.5, False),
    ("bf16 d128 causal ragged 1000 sharp", BF16, (1, 3, 1000, 128), (1, 3, 1000, 128), (1, 3, 1000, 128), True, 2.0, True),
    ("bf16 d64 full 2048", BF16, (1, 2, 2048, 64), (1, 2, 2048, 64), (1, 2, 2048, 64), False, 1.0, False),
    ("bf16 d64 causal 256 batch", BF16, (4, 8, 256, 64), (4, 8, 256, 64), (4, 8, 256, 64), True, 1.0, False),
    ("bf16 d128 rect 129x257", BF16, (3, 129, 128), (3, 257, 128), (3, 257, 128), False, 1.0, False),
    ("bf16 d64 one row", BF16, (2, 1, 64), (2, 300, 64), (2, 300, 64), False, 1.0, False),
    ("f16 d64 causal 384", np.float16, (2, 384, 64), (2, 384, 64), (2, 384, 64), True, 1.0, False),
    ("f16 d128 full 200", np.float16, (2, 200, 128), (2, 200, 128), (2, 200, 128), False, 1.0, False),
    ("f32 d64 causal 300", np.float32, (2, 300, 64), (2, 300, 64), (2, 300, 64), True, 1.0, False),
    ("f32 d128 full 130", np.float32, (130, 128), (130, 128), (130, 128), False, 1.0, False),
    ("bf16 d32 causal (zero-padded in the 64 kernel)", BF16, (2, 2, 200, 32), (2, 2, 200, 32), (2, 2, 200, 32), True, 1.0, False),
    ("bf16 d96 full 300 (zero-padded in the 128 kernel)", BF16, (3, 300, 96), (3, 300, 96), (3, 300, 96), False, 1.0, False),
    ("f16 d80 causal 257", np.float16, (2, 257, 80), (2, 257, 80), (2, 257, 80), True, 1.0, False),
    ("bf16 d8 causal 130", BF16, (2, 130, 8), (2, 130, 8), (2, 130, 8), True, 1.0, False),
    ("bf16 d96 one row against 300 keys", BF16, (2, 1, 96), (2, 300, 96), (2, 300, 96), False, 1.0, False),
    ("bf16 d20 causal (general path)", BF16, (2, 2, 200, 20), (2, 2, 200, 20), (2, 2, 200, 20), True, 1.0, False),
    ("bf16 hd 64 hd_v 128 (both in the 128 kernel)", BF16, (2, 150, 64), (2, 150, 64), (2, 150, 128), False, 1.0, False),
    ("bf16 hd 128 hd_v 64 rect 100x260", BF16, (2, 100, 128), (2, 260, 128), (2, 260, 64), False, 1.0, False),
    ("f16 hd 48 hd_v 24 causal 200", np.float16, (3, 200, 48), (3, 200, 48), (3, 200, 24), True, 1.0, False),
    ("f64 d40", np.float64, (2, 70, 40), (2, 70, 40), (2, 70, 24), True, 1.0, False),
]


@pytest.mark.parametrize("case", ORACLE_CASES, ids=[c[0] for c in ORACLE_CASES])
def test_kernels_match_oracle(case, dev):
    import limn_standin as host

    _, dtype, qs, ks, vs, causal, mul, uniform = case
    q, k, v, do = _random_case(100 + len(qs) + qs[-2], dtype, qs, ks, vs, mul, uniform)
    name = np.dtype(dtype).name
    att = host.Attention(dev, q, k, v, causal=causal)
    out, lse = att.forward()
    scale = qs[-1] ** -0.5
    want_out, want_lse = oracle.sdpa_forward(q, k, v, causal=causal, scale=scale)
    close(out, want_out, FWD_TOL[name], "O")
    close(lse, want_lse, LSE_TOL if name != "float64" else 1e-11, "L")
    # the backward kernels read the device's own O and L, as they do under autograd
    dq, dk, dv = att.backward(do)
    delta = oracle.row_delta(do, want_out)
    want_dq = oracle.sdpa_backward_q(q, k, v, do, want_lse, delta, causal=causal, scale=scale)
    want_dk, want_dv = oracle.sdpa_backward_kv(q, k, v, do, want_lse, delta, causal=causal, scale=scale)
    for got, want, what in ((dq, want_dq, "dQ"), (dk, want_dk, "dK"), (dv, want_dv, "dV")):
        close(got, want, BWD_TOL[name], what)


@pytest.mark.parametrize("t", list(range(1, 12)) + [63, 64, 65, 127, 128, 129, 255, 256, 257, 383, 385])
def test_every_tail_length_d64_bf16(t, dev):
    """Sequence lengths around every tile edge, causal and full, through the tensor-core path."""
    import limn_standin as host

    for causal in (True, False):
        q, k, v, do = _random_case(t, BF16, (2, t, 64), (2, t, 64), (2, t, 64))
        att = host.Attention(dev, q, k, v, causal=causal)
        out, lse = att.forward()
        want_out, want_lse = oracle.sdpa_forward(q, k, v, causal=causal, scale=0.125)
        close(out, want_out, 2e-2, f"t={t} causal={causal} O")
        close(lse, want_lse, LSE_TOL, f"t={t} causal={causal} L")
        dq, dk, dv = att.backward(do)
        delta = oracle.row_delta(do, want_out)
        close(dq, oracle.sdpa_backward_q(q, k, v, do, want_lse, delta, causal=causal, scale=0.125), 2e-2, f"t={t} dQ")
        want_dk, want_dv = oracle.sdpa_backward_kv(q, k, v, do, want_lse, delta, causal=causal, scale=0.125)
        close(dk, want_dk, 2e-2, f"t={t} dK")
        close(dv, want_dv, 2e-2, f"t={t} dV")


@pytest.mark.parametrize("hd", list(range(8, 129, 8)))
def test_every_head_dim_that_is_a_multiple_of_8(hd, dev):
    """bf16 heads of 8, 16, ..., 128 columns through the tensor-core kernels (built for 64 and 128; the others run
    zero-padded in the next of the two): forward and both backward kernels against the oracle, causal, a ragged
    length, with the operands of the neighbouring problem lying right behind every row's last column."""
    import limn_standin as host
    from limn_b200._lib import PATH_TCGEN05, lib

    t = 150
    assert lib().limn_b200_sdpa_path(2, 3, t, t, hd, hd, 1, 0, hd**-0.5) == PATH_TCGEN05
    q, k, v, do = _random_case(500 + hd, BF16, (3, t, hd), (3, t, hd), (3, t, hd))
    scale = hd**-0.5
    att = host.Attention(dev, q, k, v, causal=True)
    out, lse = att.forward()
    want_out, want_lse = oracle.sdpa_forward(q, k, v, causal=True, scale=scale)
    close(out, want_out, 2e-2, f"hd={hd} O")
    close(lse, want_lse, LSE_TOL, f"hd={hd} L")
    dq, dk, dv = att.backward(do)
    delta = oracle.row_delta(do, want_out)
    close(dq, oracle.sdpa_backward_q(q, k, v, do, want_lse, delta, causal=True, scale=scale), 2e-2, f"hd={hd} dQ")
    want_dk, want_dv = oracle.sdpa_backward_kv(q, k, v, do, want_lse, delta, causal=True, scale=scale)
    close(dk, want_dk, 2e-2, f"hd={hd} dK")
    close(dv, want_dv, 2e-2, f"hd={hd} dV")


MASK_CASES = [
    # id, shape (q = k = v), causal, mask kind
    ("d64 full, keys hidden at random", (2, 3, 300, 64), False, "holes"),
    ("d128 causal, padded batch", (3, 384, 128), True, "pad"),
    ("d128 full, padded batch, ragged", (2, 200, 128), False, "pad"),
    ("d64 causal, keys hidden at random", (2, 2, 257, 64), True, "holes"),
    ("d96 causal, keys hidden at random (zero-padded head)", (2, 2, 257, 96), True, "holes"),
]


@pytest.mark.parametrize("case", MASK_CASES, ids=[c[0] for c in MASK_CASES])
@pytest.mark.parametrize("dtype", [BF16, np.float16], ids=["bf16", "f16"])
def test_key_mask_on_the_tensor_core_path(case, dtype, dev):
    """A key mask with 16-bit storage: same kernels, hidden keys as -inf scores; dK and dV of a hidden key
    are exact zeros (the reference's own test of that: tests/test_attention.py:112-119 there)."""
    import limn_standin as host

    _, shape, causal, kind = case
    rng = np.random.default_rng(len(shape) * 1000 + shape[-2])
    q, k, v, do = (rng.standard_normal(shape).astype(np.float32).astype(dtype) for _ in range(4))
    t_k = shape[-2]
    if kind == "holes":
        mask = (rng.random(shape[:-1]) > 0.3).astype(np.float32)
        mask[..., 0] = 1  # under causal, row 0 sees key 0 only
    else:
        mask = np.broadcast_to((np.arange(t_k) < t_k * 2 // 3).astype(np.float32), shape[:-1]).copy()
    mask = mask.astype(dtype)
    scale = shape[-1] ** -0.5
    name = "bfloat16" if dtype == BF16 else "float16"
    att = host.Attention(dev, q, k, v, causal=causal, key_mask=mask)
    out, lse = att.forward()
    want_out, want_lse = oracle.sdpa_forward(q, k, v, mask, causal=causal, scale=scale)
    close(out, want_out, FWD_TOL[name], "O")
    close(lse, want_lse, LSE_TOL, "L")
    dq, dk, dv = att.backward(do)
    delta = oracle.row_delta(do, want_out)
    want_dq = oracle.sdpa_backward_q(q, k, v, do, want_lse, delta, mask, causal=causal, scale=scale)
    want_dk, want_dv = oracle.sdpa_backward_kv(q, k, v, do, want_lse, delta, mask, causal=causal, scale=scale)
    for got, want, what in ((dq, want_dq, "dQ"), (dk, want_dk, "dK"), (dv, want_dv, "dV")):
        close(got, want, BWD_TOL[name], what)
    hidden = mask.astype(np.float32) == 0
    assert (dk.astype(np.float32)[hidden] == 0).all() and (dv.astype(np.float32)[hidden] == 0).all()


def test_masked_row_without_a_visible_key_on_the_tensor_core_path(dev):
    """Causal with the first 5 keys hidden: rows 0-4 see nothing and come back NaN with L = -inf, the rest
    are ordinary (limn/sdpa.py:111-112)."""
    import limn_standin as host

    rng = np.random.default_rng(77)
    q, k, v = (rng.standard_normal((2, 200, 64)).astype(np.float32).astype(BF16) for _ in range(3))
    mask = np.ones((2, 200), np.float32)
    mask[:, :5] = 0
    out, lse = host.Attention(dev, q, k, v, causal=True, key_mask=mask.astype(BF16)).forward()
    want_out, want_lse = oracle.sdpa_forward(q, k, v, mask.astype(BF16), causal=True, scale=0.125)
    assert np.isnan(out.astype(np.float32)[:, :5]).all() and np.isneginf(lse[:, :5]).all()
    assert oracle.worst(out.astype(np.float32)[:, 5:], want_out.astype(np.float32)[:, 5:]) <= 2e-2
    assert float(np.abs(lse[:, 5:] - want_lse[:, 5:]).max()) <= 1e-3


def test_the_fused_dq_entry_picks_its_way_by_size():
    """limn_b200_sdpa_bwd_q_fused computes the row statistic inside the dQ kernel up to 512 keys (one launch) and runs
    the row-dot kernel in front of the plain dQ kernel beyond (two launches); delta and dQ are the same either way."""
    from limn_b200 import runtime
    from limn_b200._lib import check, lib

    L = lib()
    rng = np.random.default_rng(9)
    for t, launches in ((512, 1), (640, 2)):
        q, k, v, do = (runtime.upload(rng.standard_normal((2, t, 64)).astype(np.float32).astype(BF16)) for _ in range(4))
        out, dq_a, dq_b = (runtime.empty(2 * t * 64 * 2) for _ in range(3))
        lse, delta_a, delta_b = (runtime.empty(2 * t * 4) for _ in range(3))
        tail = (2, 2, t, t, 64, 64, 1, 0.125, None)
        check(L.limn_b200_sdpa_fwd(q.ptr, k.ptr, v.ptr, None, out.ptr, lse.ptr, *tail), "sdpa")
        check(L.limn_b200_sdpa_bwd_q_fused(q.ptr, k.ptr, v.ptr, out.ptr, do.ptr, lse.ptr, None, dq_a.ptr, delta_a.ptr, *tail), "fused dq")
        assert L.limn_b200_last_launch_count() == launches, t
        check(L.limn_b200_sdpa_delta(out.ptr, do.ptr, delta_b.ptr, 2, 2 * t, 64, None), "row dot")
        check(L.limn_b200_sdpa_bwd_q(q.ptr, k.ptr, v.ptr, do.ptr, lse.ptr, delta_b.ptr, None, dq_b.ptr, *tail), "dq")
        runtime.synchronize()
        assert runtime.device_status() == 0
        got = runtime.download(dq_a, BF16, (2, t, 64)).astype(np.float32)
        want = runtime.download(dq_b, BF16, (2, t, 64)).astype(np.float32)
        np.testing.assert_allclose(got, want, rtol=2**-7, atol=2e-3)
        np.testing.assert_allclose(runtime.download(delta_a, np.float32, (2, t)), runtime.download(delta_b, np.float32, (2, t)), rtol=1e-5, atol=1e-5)


TILED_CASES = [
    # id, dtype, q, k, v shapes, causal, mask kind
    ("f32 d64 causal 256 batch (a GPT layer in float32)", np.float32, (4, 8, 256, 64), (4, 8, 256, 64), (4, 8, 256, 64), True, None),
    ("f32 d128 causal ragged 1000", np.float32, (2, 1000, 128), (2, 1000, 128), (2, 1000, 128), True, None),
    ("f32 d37 full 131 (rows that are no whole 16-byte pieces)", np.float32, (3, 131, 37), (3, 131, 37), (3, 131, 37), False, None),
    ("f32 d40 hd_v 24 rect 70x333", np.float32, (2, 70, 40), (2, 333, 40), (2, 333, 24), False, None),
    ("f32 d64 causal, keys hidden at random", np.float32, (2, 2, 257, 64), (2, 2, 257, 64), (2, 2, 257, 64), True, "holes"),
    ("f32 d128 full, padded batch", np.float32, (3, 200, 128), (3, 200, 128), (3, 200, 128), False, "pad"),
    ("f32 d32 rect 16x16 (the smallest tiled sides)", np.float32, (5, 16, 32), (5, 16, 32), (5, 16, 32), False, None),
    ("f32 d256 causal 300", np.float32, (2, 300, 256), (2, 300, 256), (2, 300, 256), True, None),
    ("bf16 d192 hd_v 128 full 200, keys hidden at random", BF16, (2, 200, 192), (2, 200, 192), (2, 200, 128), False, "holes"),
    ("f16 d100 causal 300", np.float16, (2, 300, 100), (2, 300, 100), (2, 300, 100), True, None),
    ("bf16 d36 full 500, padded batch", BF16, (2, 500, 36), (2, 500, 36), (2, 500, 36), False, "pad"),
    ("bf16 hd 100 hd_v 60 rect 100x260", BF16, (2, 100, 100), (2, 260, 100), (2, 260, 60), False, None),
]


@pytest.mark.parametrize("case", TILED_CASES, ids=[c[0] for c in TILED_CASES])
def test_tiled_general_kernels_match_oracle(case, dev):
    """What the tensor-core kernels do not take and still fills a tile: float32 at its own width, head dims other
    than 64 and 128 up to 128, hd != hd_v; with masks, ragged and rectangular sides. Hidden keys get exact-zero
    dK and dV, and a second run gives the same bits (one owner per total, fixed summation order)."""
    import limn_standin as host
    from limn_b200._lib import PATH_GENERAL, lib

    _, dtype, qs, ks, vs, causal, kind = case
    name = "bfloat16" if dtype == BF16 else np.dtype(dtype).name
    code = {"float32": 0, "float16": 1, "bfloat16": 2}[name]
    assert lib().limn_b200_sdpa_path(code, int(np.prod(qs[:-2])), qs[-2], ks[-2], qs[-1], vs[-1], int(causal), int(kind is not None), qs[-1] ** -0.5) == PATH_GENERAL
    q, k, v, do = _random_case(300 + qs[-2] + qs[-1], dtype, qs, ks, vs)
    mask = None
    if kind is not None:
        rng = np.random.default_rng(qs[-2])
        t_k = ks[-2]
        if kind == "holes":
            mask = (rng.random(ks[:-1]) > 0.3).astype(np.float32)
            mask[..., 0] = 1  # under causal, row 0 sees key 0 only
        else:
            mask = np.broadcast_to((np.arange(t_k) < t_k * 2 // 3).astype(np.float32), ks[:-1]).copy()
        mask = mask.astype(dtype)
    scale = qs[-1] ** -0.5
    att = host.Attention(dev, q, k, v, causal=causal, key_mask=mask)
    out, lse = att.forward()
    want_out, want_lse = oracle.sdpa_forward(q, k, v, mask, causal=causal, scale=scale)
    close(out, want_out, FWD_TOL[name], "O")
    close(lse, want_lse, LSE_TOL, "L")
    dq, dk, dv = att.backward(do)
    delta = oracle.row_delta(do, want_out)
    want_dq = oracle.sdpa_backward_q(q, k, v, do, want_lse, delta, mask, causal=causal, scale=scale)
    want_dk, want_dv = oracle.sdpa_backward_kv(q, k, v, do, want_lse, delta, mask, causal=causal, scale=scale)
    for got, want, what in ((dq, want_dq, "dQ"), (dk, want_dk, "dK"), (dv, want_dv, "dV")):
        close(got, want, BWD_TOL[name], what)
    if mask is not None:
        hidden = mask.astype(np.float32) == 0
        assert (dk.astype(np.float32)[hidden] == 0).all() and (dv.astype(np.float32)[hidden] == 0).all()
    again = host.Attention(dev, q, k, v, causal=causal, key_mask=mask)
    out2, lse2 = again.forward()
    assert out2.tobytes() == out.tobytes() and lse2.tobytes() == lse.tobytes()
    for first, second in zip((dq, dk, dv), again.backward(do)):
        assert first.tobytes() == second.tobytes()


def test_tiled_general_kernels_on_rows_without_a_visible_key(dev):
    """float32, causal with the first 5 keys hidden: rows 0-4 see nothing and come back NaN with L = -inf, the
    rest are ordinary, and dQ of the empty rows is zero (limn/sdpa.py:111-112)."""
    import limn_standin as host

    rng = np.random.default_rng(78)
    q, k, v, do = (rng.standard_normal((2, 200, 64)).astype(np.float32) for _ in range(4))
    mask = np.ones((2, 200), np.float32)
    mask[:, :5] = 0
    att = host.Attention(dev, q, k, v, causal=True, key_mask=mask)
    out, lse = att.forward()
    want_out, want_lse = oracle.sdpa_forward(q, k, v, mask, causal=True, scale=0.125)
    assert np.isnan(out[:, :5]).all() and np.isneginf(lse[:, :5]).all()
    assert oracle.worst(out[:, 5:], want_out[:, 5:]) <= 1e-4
    assert float(np.abs(lse[:, 5:] - want_lse[:, 5:]).max()) <= 1e-3


FUSED_CASES = [
    # id, dtype, code, shape (q = k = v), causal, key mask?, layout
    ("bf16 d128 causal", BF16, 2, (3, 384, 128), True, False, "bhtd"),
    ("bf16 d64 full ragged", BF16, 2, (2, 200, 64), False, False, "bhtd"),
    ("f16 d64 causal masked", np.float16, 1, (4, 300, 64), True, True, "bhtd"),
    ("bf16 d128 full token-major", BF16, 2, (6, 260, 128), False, False, "bthd"),
    ("bf16 d96 causal (zero-padded head)", BF16, 2, (3, 300, 96), True, False, "bhtd"),
    ("f16 d40 full token-major (zero-padded head)", np.float16, 1, (4, 200, 40), False, False, "bthd"),
    ("f32 d32 causal (general path)", np.float32, 0, (2, 100, 32), True, False, "bhtd"),
]


@pytest.mark.parametrize("case", FUSED_CASES, ids=[c[0] for c in FUSED_CASES])
def test_fused_dq_matches_delta_then_dq(case):
    """limn_b200_sdpa_bwd_q_fused computes the row dot inside the dQ pass and leaves it for the dK/dV pass: its dQ
    and its delta must be what limn_b200_sdpa_delta followed by limn_b200_sdpa_bwd_q give, and delta the oracle's."""
    from limn_b200 import runtime
    from limn_b200._lib import check, lib

    L = lib()
    _, dtype, code, shape, causal, masked, layout = case
    bh, t, d = shape
    rng = np.random.default_rng(bh * 1000 + t)
    q, k, v, do = (rng.standard_normal(shape).astype(np.float32).astype(dtype) for _ in range(4))
    dev = [runtime.upload(a) for a in (q, k, v, do)]
    mask = runtime.upload(np.broadcast_to(np.arange(t) < t * 3 // 4, (bh, t)).astype(np.float32).astype(dtype)) if masked else None
    m = mask.ptr if mask is not None else None
    out, lse = runtime.empty(q.nbytes), runtime.empty(bh * t * 4)
    delta_a, delta_b = runtime.empty(bh * t * 4), runtime.empty(bh * t * 4)
    dq_a, dq_b = runtime.empty(q.nbytes), runtime.empty(q.nbytes)
    if layout == "bthd":
        # the same bytes read as one batch of bh heads held token-major: (1, t, bh, d)
        tail = (1, code, 1, bh, t, t, d, d, int(causal), d**-0.5, None)
        check(L.limn_b200_sdpa_fwd_layout(dev[0].ptr, dev[1].ptr, dev[2].ptr, m, out.ptr, lse.ptr, *tail), "sdpa")
        check(L.limn_b200_sdpa_delta_layout(out.ptr, dev[3].ptr, delta_a.ptr, 1, code, 1, bh, t, d, None), "row dot")
        check(L.limn_b200_sdpa_bwd_q_layout(dev[0].ptr, dev[1].ptr, dev[2].ptr, dev[3].ptr, lse.ptr, delta_a.ptr, m, dq_a.ptr, *tail), "dq")
        check(L.limn_b200_sdpa_bwd_q_fused_layout(dev[0].ptr, dev[1].ptr, dev[2].ptr, out.ptr, dev[3].ptr, lse.ptr, m, dq_b.ptr, delta_b.ptr, *tail), "fused dq")
    else:
        tail = (code, bh, t, t, d, d, int(causal), d**-0.5, None)
        check(L.limn_b200_sdpa_fwd(dev[0].ptr, dev[1].ptr, dev[2].ptr, m, out.ptr, lse.ptr, *tail), "sdpa")
        check(L.limn_b200_sdpa_delta(out.ptr, dev[3].ptr, delta_a.ptr, code, bh * t, d, None), "row dot")
        check(L.limn_b200_sdpa_bwd_q(dev[0].ptr, dev[1].ptr, dev[2].ptr, dev[3].ptr, lse.ptr, delta_a.ptr, m, dq_a.ptr, *tail), "dq")
        check(L.limn_b200_sdpa_bwd_q_fused(dev[0].ptr, dev[1].ptr, dev[2].ptr, out.ptr, dev[3].ptr, lse.ptr, m, dq_b.ptr, delta_b.ptr, *tail), "fused dq")
    assert L.limn_b200_last_launch_count() == (1 if code != 0 else 2)  # the general family still runs the row dot as a kernel
    assert runtime.device_status() == 0
    two_step, fused = runtime.download(delta_a, np.float32, (bh, t)), runtime.download(delta_b, np.float32, (bh, t))
    np.testing.assert_allclose(fused, two_step, rtol=1e-5, atol=1e-5 * float(np.abs(two_step).max()))
    device_out = runtime.download(out, dtype, (bh, t, d) if layout == "bhtd" else (t, bh, d))
    do_as_held = do if layout == "bhtd" else do.reshape(t, bh, d)
    want_delta = oracle.row_delta(do_as_held, device_out)[..., 0]
    parity(fused, want_delta if layout == "bhtd" else want_delta.T, 1e-5, "fused delta")
    a, b = widen(runtime.download(dq_a, dtype, shape)), widen(runtime.download(dq_b, dtype, shape))
    np.testing.assert_allclose(b, a, rtol=2**-7 if code != 0 else 1e-5, atol=2e-3 if code != 0 else 1e-5)


DECODE_CASES = [
    # id, dtype, code, bh, t_q, t_k, d, key mask kind, layout
    ("bf16 d128 one row 4096 keys", BF16, 2, 24, 1, 4096, 128, None, "bhtd"),
    ("bf16 d64 one row ragged 1000", BF16, 2, 7, 1, 1000, 64, None, "bhtd"),
    ("f16 d128 four rows 300 keys", np.float16, 1, 5, 4, 300, 128, None, "bhtd"),
    ("f16 d64 three rows, padded cache", np.float16, 1, 6, 3, 515, 64, "pad", "bhtd"),
    ("bf16 d128 two rows, holes", BF16, 2, 4, 2, 777, 128, "holes", "bhtd"),
    ("bf16 d64 one row, token-major", BF16, 2, 12, 1, 640, 64, None, "bthd"),
    ("bf16 d128 one row, 3 keys", BF16, 2, 3, 1, 3, 128, None, "bhtd"),
    ("bf16 d128 one row, 400 problems (one CTA each)", BF16, 2, 400, 1, 513, 128, None, "bhtd"),
    ("bf16 d64 two rows, 80 problems (clusters of 2)", BF16, 2, 80, 2, 2048, 64, "pad", "bhtd"),
]


@pytest.mark.parametrize("case", DECODE_CASES, ids=[c[0] for c in DECODE_CASES])
def test_decode_shapes_on_the_streaming_kernel(case):
    """A few query rows against many keys (the step of a kv cache; the reference's own test of the shape is
    tests/test_attention.py:385-396 there): served by the bandwidth-bound decode kernel, checked against the oracle,
    twice for the bits."""
    from limn_b200 import runtime
    from limn_b200._lib import PATH_DECODE, check, lib

    L = lib()
    _, dtype, code, bh, t_q, t_k, d, mask_kind, layout = case
    assert L.limn_b200_sdpa_path(code, bh, t_q, t_k, d, d, 0, int(mask_kind is not None), d**-0.5) == PATH_DECODE
    rng = np.random.default_rng(bh * 100 + t_k)
    q = rng.standard_normal((bh, t_q, d)).astype(np.float32).astype(dtype)
    k, v = (rng.standard_normal((bh, t_k, d)).astype(np.float32).astype(dtype) for _ in range(2))
    mask = None
    if mask_kind == "pad":
        mask = np.broadcast_to(np.arange(t_k) < t_k * 2 // 3, (bh, t_k)).astype(np.float32).astype(dtype)
    elif mask_kind == "holes":
        mask = (rng.random((bh, t_k)) > 0.4).astype(np.float32).astype(dtype)
        mask[-1] = 0  # the last problem sees no key at all: NaN rows, L = -inf
    held = [np.ascontiguousarray(a if layout == "bhtd" else a.transpose(1, 0, 2)) for a in (q, k, v)]  # (t, bh, d) = one batch of bh heads
    dev = [runtime.upload(a) for a in held]
    mask_dev = runtime.upload(mask) if mask is not None else None
    results = []
    for _ in range(2):
        out, lse = runtime.empty(q.nbytes), runtime.empty(bh * t_q * 4)
        m = mask_dev.ptr if mask_dev is not None else None
        if layout == "bthd":
            check(L.limn_b200_sdpa_fwd_layout(dev[0].ptr, dev[1].ptr, dev[2].ptr, m, out.ptr, lse.ptr, 1, code, 1, bh, t_q, t_k, d, d, 0, d**-0.5, None), "sdpa")
        else:
            check(L.limn_b200_sdpa_fwd(dev[0].ptr, dev[1].ptr, dev[2].ptr, m, out.ptr, lse.ptr, code, bh, t_q, t_k, d, d, 0, d**-0.5, None), "sdpa")
        got = runtime.download(out, dtype, (bh, t_q, d) if layout == "bhtd" else (t_q, bh, d))
        results.append((got if layout == "bhtd" else got.transpose(1, 0, 2), runtime.download(lse, np.float32, (bh, t_q, 1))))
    assert runtime.device_status() == 0
    want_out, want_lse = oracle.sdpa_forward(q, k, v, mask, causal=False, scale=d**-0.5)
    name = "bfloat16" if dtype == BF16 else "float16"
    parity(results[0][0], want_out, FWD_TOL[name], f"decode {case[0]} O")
    parity(results[0][1], want_lse, LSE_TOL, f"decode {case[0]} L")
    if mask_kind == "holes":
        assert np.isnan(widen(results[0][0][-1])).all() and np.isneginf(results[0][1][-1]).all()
    for a, b in zip(results[0], results[1], strict=True):
        np.testing.assert_array_equal(np.ascontiguousarray(a).view(np.uint8), np.ascontiguousarray(b).view(np.uint8))


def test_two_runs_give_the_same_bits(dev):
    import limn_standin as host

    for dtype, shape in ((BF16, (2, 2, 300, 128)), (np.float32, (2, 3, 64, 16))):
        q, k, v, do = _random_case(5, dtype, shape, shape, shape)
        runs = []
        for _ in range(2):
            att = host.Attention(dev, q, k, v, causal=True)
            out, lse = att.forward()
            runs.append((out, lse, *att.backward(do)))
        for first, second in zip(*runs, strict=True):
            np.testing.assert_array_equal(first.view(np.uint8), second.view(np.uint8))


def test_work_counters_come_back_to_zero_launch_after_launch(dev):
    """The tensor-core kernels' CTAs fetch their work items from a counter pair that the last CTA zeroes again;
    the pairs are handed out from a ring of 128. More launches than the ring has pairs, with more items than
    the GPU has SMs (600 > 148) and with fewer, must all give the first launch's bits."""
    import limn_standin as host

    for shape in ((150, 2, 200, 64), (3, 1, 300, 128)):
        q, k, v, do = _random_case(21, BF16, shape, shape, shape)
        first = None
        for _ in range(50):  # 3 tensor-core launches per round and shape: 300 in all
            att = host.Attention(dev, q, k, v, causal=True)
            out, lse = att.forward()
            got = (out, lse, *att.backward(do))
            if first is None:
                first = got
                want = oracle.sdpa_forward(q[:1], k[:1], v[:1], causal=True, scale=shape[-1] ** -0.5)[0]
                assert np.abs(widen(out[:1]) - widen(want)).max() <= 2e-2
            else:
                for a, b in zip(first, got, strict=True):
                    np.testing.assert_array_equal(a.view(np.uint8), b.view(np.uint8))
        dev.finish()


def test_hidden_keys_get_exactly_zero_gradients(dev):
    import limn_standin as host

    q, k, v, do = _random_case(9, np.float32, (2, 3, 32, 8), (2, 3, 32, 8), (2, 3, 32, 12))
    mask = np.broadcast_to(np.arange(32) < 20, (2, 3, 32)).astype(np.float32)
    att = host.Attention(dev, q, k, v, causal=True, key_mask=mask)
    att.forward()
    _, dk, dv = att.backward(do)
    assert (dk[..., 20:, :] == 0).all() and (dv[..., 20:, :] == 0).all()
    assert np.abs(dk[..., :20, :]).min() > 0


def test_row_without_a_visible_key_is_nan_with_minus_inf_lse(dev):
    import limn_standin as host

    q, k, v, _ = _random_case(10, np.float32, (2, 8, 4), (2, 8, 4), (2, 8, 4))
    mask = np.ones((2, 8), np.float32)
    mask[1] = 0
    out, lse = host.Attention(dev, q, k, v, key_mask=mask).forward()
    assert np.isfinite(out[0]).all() and np.isnan(out[1]).all()
    assert np.isneginf(lse[1]).all()


def test_tensor_core_path_is_the_one_that_serves_the_tuned_shapes():
    from limn_b200._lib import PATH_GENERAL, PATH_TCGEN05, lib

    path = lib().limn_b200_sdpa_path
    assert path(2, 256, 4096, 4096, 128, 128, 1, 0, 128**-0.5) == PATH_TCGEN05
    assert path(2, 256, 256, 256, 64, 64, 1, 0, 0.125) == PATH_TCGEN05
    assert path(1, 4, 100, 300, 64, 64, 0, 0, 0.125) == PATH_TCGEN05
    from limn_b200._lib import PATH_DECODE

    assert path(2, 64, 1, 4096, 128, 128, 0, 1, 128**-0.5) == PATH_DECODE  # a few query rows, no causal mask
    assert path(2, 64, 4, 4096, 64, 64, 0, 0, 0.125) == PATH_DECODE
    assert path(2, 64, 5, 4096, 64, 64, 0, 0, 0.125) == PATH_TCGEN05
    assert path(2, 64, 1, 1, 64, 64, 1, 0, 0.125) == PATH_TCGEN05  # causal is a prefill shape, however short
    assert path(0, 2, 128, 128, 32, 32, 1, 0, 32**-0.5) == PATH_GENERAL
    assert path(2, 2, 128, 128, 64, 64, 0, 1, 0.125) == PATH_TCGEN05  # a key mask stays on the tensor-core path
    assert path(0, 2, 128, 128, 64, 64, 0, 1, 0.125) == PATH_GENERAL


def test_launch_errors_surface_as_runtime_errors(dev):
    import limn_standin as host

    with pytest.raises(ValueError, match="square keys"):
        host.Attention(dev, np.zeros((4, 8), np.float32), np.zeros((5, 8), np.float32), np.zeros((5, 8), np.float32), causal=True)
    lib = __import__("limn_b200._lib", fromlist=["lib"]).lib()
    assert lib.limn_b200_sdpa_fwd(None, None, None, None, None, None, 0, 1, 4, 4, 8, 8, 0, 1.0, None) == 1
    assert b"null" in lib.limn_b200_last_error()
