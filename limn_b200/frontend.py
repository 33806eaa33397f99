"""An optional change to limn's frontend: the row dot of the attention backward folded into the dQ kernel.

limn's autograd computes delta = sum_d dO * O between the forward and the two backward CUSTOM ops as ordinary
graph work (limn/tensor.py:702-707): a reduce kernel of its own, scheduled by limn, whose result both backward
ops read. The library's dQ kernel can compute that statistic for the query rows it owns on the way
(limn_b200_sdpa_bwd_q_fused) and leave it for the dK/dV kernel, which saves the reduce, one pass over O and dO
and one launch per attention layer and step.

`fuse_row_dot()` makes limn use it. It replaces `limn.tensor._attention_backward` (the function
`Tensor.attention` calls for its grad_fn, limn/tensor.py:569-574, :679-714) with one that builds

    custom("sdpa_bwd_q_fused", (q, k, v, O, dO, L[, mask]))  ->  (dQ, delta)
    custom("sdpa_bwd_kv",      (q, k, v, dO, L, delta[, mask])) ->  (dK, dV)

whenever the active device registers "sdpa_bwd_q_fused" (limn_b200.install() does), and falls back to limn's
own function everywhere else: on the numpy and c devices, when the gradient is itself being differentiated,
and on a cuda device without these kernels. Nothing else in limn changes; as a patch to limn's source it is
the dozen lines of `backward` below in place of limn/tensor.py:702-711.
"""

from __future__ import annotations

from collections.abc import Callable

SDPA_BWD_Q_FUSED = "sdpa_bwd_q_fused"


def fuse_row_dot() -> Callable[[], None]:
    """Patch limn's frontend as described above; returns a function that undoes it."""
    import limn.tensor as frontend
    from limn import sdpa
    from limn.ops import custom

    original = frontend._attention_backward
    if getattr(original, "_limn_b200_fused", False):
        return lambda: None

    def _attention_backward(out, lse, q, k, v, mask, *, causal, scale):
        limns_own = original(out, lse, q, k, v, mask, causal=causal, scale=scale)

        def backward(g):
            active = frontend.device.active()
            if frontend.grad_enabled or not (active.has_custom(SDPA_BWD_Q_FUSED) and active.has_custom(sdpa.SDPA_BWD_KV)):
                return limns_own(g)
            do = frontend._contiguous(g)
            tail = (mask,) if mask is not None else ()
            params = (causal, scale)
            dq, delta = custom(SDPA_BWD_Q_FUSED, tuple(t.node for t in (q, k, v, out, do, lse) + tail), params,
                               ((q.dtype, q.shape), (lse.dtype, lse.shape)))
            held = (q, k, v, do, lse, frontend.Tensor.from_node(delta)) + tail
            dk, dv = custom(sdpa.SDPA_BWD_KV, tuple(t.node for t in held), params, ((k.dtype, k.shape), (v.dtype, v.shape)))
            return frontend.Tensor.from_node(dq), frontend.Tensor.from_node(dk), frontend.Tensor.from_node(dv)

        return backward

    _attention_backward._limn_b200_fused = True  # type: ignore[attr-defined]
    frontend._attention_backward = _attention_backward

    def undo() -> None:
        frontend._attention_backward = original

    return undo
