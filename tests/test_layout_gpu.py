"""The layout entry points: operands held as (batch, t, heads, hd), read and written in place.

limn's frontend permutes such activations to (batch, heads, t, hd) and copies them dense before
every attention call (limn/tensor.py:561-562). The *_layout entry points reach the same rows
through the tensor maps' strides instead. The check is that they give, bit for bit, what the
dense entry points give on the permuted copies (every row is accumulated in the same order
either way), that the dense layout code is the dense entry point, and that one case also
matches the CPU oracle."""

from __future__ import annotations

import numpy as np
import pytest
from conftest import BF16, widen

from oracle import sdpa_oracle as oracle

pytestmark = pytest.mark.gpu

CASES = [
    # batch, heads, t_q, t_k, hd, causal, dtype
    (2, 3, 300, 300, 64, True, BF16),
    (1, 5, 257, 257, 128, True, BF16),
    (2, 2, 130, 390, 128, False, np.dtype(np.float16)),
    (3, 4, 128, 128, 64, False, BF16),
    (2, 3, 200, 200, 96, True, BF16),  # narrower heads run zero-padded in the 128 and the 64 kernel
    (2, 2, 150, 150, 40, False, np.dtype(np.float16)),
]


def _run(layout: str, arrays, mask, batch, heads, t_q, t_k, hd, causal, dtype):
    """forward, delta, dQ, dK/dV through the layout entry points; arrays are in `layout` order."""
    from limn_b200 import runtime
    from limn_b200._lib import DTYPE_CODES, LAYOUT_CODES, check, lib

    L = lib()
    code = DTYPE_CODES["bfloat16" if dtype == BF16 else "float16"]
    q, k, v, do = (runtime.upload(a) for a in arrays)
    m = runtime.upload(mask) if mask is not None else None
    out, dq = runtime.empty(arrays[0].nbytes), runtime.empty(arrays[0].nbytes)
    dk, dv = runtime.empty(arrays[1].nbytes), runtime.empty(arrays[1].nbytes)
    lse, delta = runtime.empty(batch * heads * t_q * 4), runtime.empty(batch * heads * t_q * 4)
    tail = (LAYOUT_CODES[layout], code, batch, heads, t_q, t_k, hd, hd, int(causal), hd**-0.5, None)
    mp = m.ptr if m is not None else None
    check(L.limn_b200_sdpa_fwd_layout(q.ptr, k.ptr, v.ptr, mp, out.ptr, lse.ptr, *tail), "sdpa")
    check(L.limn_b200_sdpa_delta_layout(out.ptr, do.ptr, delta.ptr, LAYOUT_CODES[layout], code, batch, heads, t_q, hd, None), "row dot")
    check(L.limn_b200_sdpa_bwd_q_layout(q.ptr, k.ptr, v.ptr, do.ptr, lse.ptr, delta.ptr, mp, dq.ptr, *tail), "sdpa_bwd_q")
    check(L.limn_b200_sdpa_bwd_kv_layout(q.ptr, k.ptr, v.ptr, do.ptr, lse.ptr, delta.ptr, mp, dk.ptr, dv.ptr, *tail), "sdpa_bwd_kv")
    runtime.synchronize()
    assert runtime.device_status() == 0
    shape_q, shape_k = arrays[0].shape, arrays[1].shape
    return {
        "out": runtime.download(out, dtype, shape_q),
        "lse": runtime.download(lse, np.float32, (batch, heads, t_q)),
        "delta": runtime.download(delta, np.float32, (batch, heads, t_q)),
        "dq": runtime.download(dq, dtype, shape_q),
        "dk": runtime.download(dk, dtype, shape_k),
        "dv": runtime.download(dv, dtype, shape_k),
    }


def _inputs(seed, batch, heads, t_q, t_k, hd, dtype):
    rng = np.random.default_rng(seed)
    draw = lambda t: (rng.standard_normal((batch, heads, t, hd)).astype(np.float32) * 0.7).astype(dtype)
    q, k, v = draw(t_q), draw(t_k), draw(t_k)
    do = draw(t_q)
    return q, k, v, do


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"b{c[0]}h{c[1]}q{c[2]}k{c[3]}d{c[4]}{'c' if c[5] else 'f'}{c[6].name}")
def test_token_major_operands_give_the_dense_bits(case):
    batch, heads, t_q, t_k, hd, causal, dtype = case
    dense = _inputs(31, batch, heads, t_q, t_k, hd, dtype)
    token_major = tuple(np.ascontiguousarray(a.transpose(0, 2, 1, 3)) for a in dense)
    want = _run("bhtd", dense, None, *case)
    got = _run("bthd", token_major, None, *case)
    for name in ("out", "dq", "dk", "dv"):
        back = got[name].transpose(0, 2, 1, 3)
        np.testing.assert_array_equal(back.view(np.uint16), want[name].view(np.uint16), err_msg=name)
    for name in ("lse", "delta"):
        np.testing.assert_array_equal(got[name].view(np.uint32), want[name].view(np.uint32), err_msg=name)


def test_token_major_with_a_key_mask_matches_the_oracle():
    batch, heads, t, hd = 2, 3, 200, 64
    q, k, v, do = _inputs(32, batch, heads, t, t, hd, BF16)
    mask = np.ones((batch, heads, t), np.float32)
    mask[:, :, 150:] = 0
    mask[1, 2, 1::3] = 0
    mask = mask.astype(BF16)
    token_major = tuple(np.ascontiguousarray(a.transpose(0, 2, 1, 3)) for a in (q, k, v, do))
    got = _run("bthd", token_major, mask, batch, heads, t, t, hd, True, BF16)
    scale = hd**-0.5
    out, lse = oracle.sdpa_forward(q, k, v, mask, causal=True, scale=scale)
    delta = oracle.row_delta(do, out)
    dq = oracle.sdpa_backward_q(q, k, v, do, lse, delta, mask, causal=True, scale=scale)
    dk, dv = oracle.sdpa_backward_kv(q, k, v, do, lse, delta, mask, causal=True, scale=scale)
    for name, want in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        err = np.abs(widen(got[name].transpose(0, 2, 1, 3)) - widen(want)).max()
        assert err <= 2e-2, f"{name}: {err}"
    assert np.abs(got["lse"] - lse[..., 0]).max() <= 1e-3
    assert (widen(got["dk"].transpose(0, 2, 1, 3))[:, :, 150:] == 0).all()


@pytest.mark.parametrize("hd,causal,t", [(64, True, 300), (128, False, 257), (80, True, 200)], ids=["d64 causal", "d128 full", "d80 causal"])
def test_slices_of_one_projection_buffer_give_the_dense_bits(hd, causal, t):
    """The strided entry points on what a transformer layer really holds: q, k, v as slices of one
    (batch, t, 3, heads, hd) projection output, dO and the results token-major, dK and dV written straight into a
    (batch, t, 2, heads, hd) buffer. Bit for bit what the dense entry points give on dense copies."""
    import ctypes

    from limn_b200 import runtime
    from limn_b200._lib import check, lib

    L = lib()
    batch, heads = 2, 3
    dense = _inputs(35, batch, heads, t, t, hd, BF16)
    want = _run("bhtd", dense, None, batch, heads, t, t, hd, causal, BF16)
    qkv = np.stack([a.transpose(0, 2, 1, 3) for a in dense[:3]], axis=2)  # (batch, t, 3, heads, hd)
    do = np.ascontiguousarray(dense[3].transpose(0, 2, 1, 3))               # (batch, t, heads, hd)
    qkv_dev, do_dev = runtime.upload(np.ascontiguousarray(qkv)), runtime.upload(do)
    row3, row2, row1 = 3 * heads * hd, 2 * heads * hd, heads * hd
    in_qkv = (t * row3, hd, row3)       # (batch, head, row) strides of a slice of the projection buffer
    token_major = (t * row1, hd, row1)
    in_kv_grad = (t * row2, hd, row2)
    q_ptr, k_ptr, v_ptr = (qkv_dev.ptr + i * row1 * 2 for i in range(3))
    out, dq = runtime.empty(do.nbytes), runtime.empty(do.nbytes)
    dkv = runtime.empty(2 * do.nbytes)
    lse, delta = runtime.empty(batch * heads * t * 4), runtime.empty(batch * heads * t * 4)
    arr = lambda *triples: (ctypes.c_longlong * (3 * len(triples)))(*[x for tr in triples for x in tr])
    tail = (2, batch, heads, t, t, hd, hd, int(causal), hd**-0.5, None)
    check(L.limn_b200_sdpa_fwd_strided(q_ptr, k_ptr, v_ptr, None, out.ptr, lse.ptr, arr(in_qkv, in_qkv, in_qkv, token_major), *tail), "sdpa")
    check(L.limn_b200_sdpa_bwd_q_fused_strided(q_ptr, k_ptr, v_ptr, out.ptr, do_dev.ptr, lse.ptr, None, dq.ptr, delta.ptr,
                                               arr(in_qkv, in_qkv, in_qkv, token_major, token_major, token_major), *tail), "dq")
    check(L.limn_b200_sdpa_bwd_kv_strided(q_ptr, k_ptr, v_ptr, do_dev.ptr, lse.ptr, delta.ptr, None, dkv.ptr, dkv.ptr + row1 * 2,
                                          arr(in_qkv, in_qkv, in_qkv, token_major, in_kv_grad, in_kv_grad), *tail), "dk, dv")
    runtime.synchronize()
    assert runtime.device_status() == 0
    got_out = runtime.download(out, BF16, (batch, t, heads, hd)).transpose(0, 2, 1, 3)
    got_dq = runtime.download(dq, BF16, (batch, t, heads, hd)).transpose(0, 2, 1, 3)
    got_dkv = runtime.download(dkv, BF16, (batch, t, 2, heads, hd))
    np.testing.assert_array_equal(got_out.view(np.uint16), want["out"].view(np.uint16))
    np.testing.assert_array_equal(runtime.download(lse, np.uint32, (batch, heads, t)), want["lse"].view(np.uint32))
    # the fused row dot sums in another order than the reduce kernel: gradients agree to a bfloat16 step
    for got, name in ((got_dq, "dq"), (got_dkv[:, :, 0].transpose(0, 2, 1, 3), "dk"), (got_dkv[:, :, 1].transpose(0, 2, 1, 3), "dv")):
        np.testing.assert_allclose(widen(got), widen(want[name]), rtol=2**-7, atol=2e-3, err_msg=name)
    # misuse is refused before anything is launched
    from limn_b200._lib import last_error

    bad = arr((t * row3, hd, row3 + 4), in_qkv, in_qkv, token_major)
    assert L.limn_b200_sdpa_fwd_strided(q_ptr, k_ptr, v_ptr, None, out.ptr, lse.ptr, bad, *tail) == 1 and "multiples of 8" in last_error()
    assert L.limn_b200_sdpa_fwd_strided(q_ptr, k_ptr, v_ptr, None, out.ptr, lse.ptr, None, *tail) == 1
    assert L.limn_b200_sdpa_fwd_strided(q_ptr, k_ptr, v_ptr, None, out.ptr, lse.ptr, arr(in_qkv, in_qkv, in_qkv, token_major),
                                        0, batch, heads, t, t, hd, hd, int(causal), hd**-0.5, None) == 2  # float32: not served strided


def test_dense_layout_code_is_the_dense_entry_point():
    from limn_b200 import runtime
    from limn_b200._lib import check, lib

    L = lib()
    batch, heads, t, hd = 2, 2, 160, 64
    q, k, v, _ = _inputs(33, batch, heads, t, t, hd, BF16)
    bufs = [runtime.upload(a) for a in (q, k, v)]
    outs = []
    for which in range(2):
        out, lse = runtime.empty(q.nbytes), runtime.empty(batch * heads * t * 4)
        if which == 0:
            check(L.limn_b200_sdpa_fwd(*(b.ptr for b in bufs), None, out.ptr, lse.ptr, 2, batch * heads, t, t, hd, hd, 1, hd**-0.5, None), "sdpa")
        else:
            check(L.limn_b200_sdpa_fwd_layout(*(b.ptr for b in bufs), None, out.ptr, lse.ptr, 0, 2, batch, heads, t, t, hd, hd, 1, hd**-0.5, None), "sdpa")
        outs.append((runtime.download(out, BF16, q.shape), runtime.download(lse, np.float32, (batch * heads, t))))
    np.testing.assert_array_equal(outs[0][0].view(np.uint16), outs[1][0].view(np.uint16))
    np.testing.assert_array_equal(outs[0][1], outs[1][1])


def test_token_major_refuses_what_the_tensor_core_kernels_do_not_take():
    from limn_b200 import runtime
    from limn_b200._lib import last_error, lib

    L = lib()
    a = runtime.upload(np.zeros((1, 16, 2, 32), np.float32))
    out, lse = runtime.empty(a.nbytes), runtime.empty(2 * 16 * 4)
    code = L.limn_b200_sdpa_fwd_layout(a.ptr, a.ptr, a.ptr, None, out.ptr, lse.ptr, 1, 0, 1, 2, 16, 16, 32, 32, 0, 0.2, None)
    assert code == 2 and "contiguous" in last_error()
    assert L.limn_b200_last_launch_count() == 0
