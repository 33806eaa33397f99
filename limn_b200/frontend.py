"""Two optional changes to limn's frontend: the row dot of the attention backward folded into the dQ kernel
(fuse_row_dot), and attention over the operands as the model holds them, without the copies in front of every
call (read_views_in_place).

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


# ---------------------------------------------------------------- attention over views, in place

SDPA_STRIDED = "sdpa_strided"
SDPA_BWD_Q_FUSED_STRIDED = "sdpa_bwd_q_fused_strided"
SDPA_BWD_KV_STRIDED = "sdpa_bwd_kv_strided"
STRIDED_NAMES = (SDPA_STRIDED, SDPA_BWD_Q_FUSED_STRIDED, SDPA_BWD_KV_STRIDED)


def read_views_in_place() -> Callable[[], None]:
    """Patch `Tensor.attention` so that q, k and v are handed to the kernels as the views they are.

    A transformer layer computes one projection, (batch, t, 3 * heads * hd), and takes q, k and v as
    `reshape(batch, t, 3, heads, hd).permute(2, 0, 3, 1, 4)` slices of it; limn's `Tensor.attention` then wraps
    each in CONTIGUOUS, a full copy into (batch, heads, t, hd) order, before the CUSTOM node may read it
    (limn/tensor.py:561-562, :736-746), and the layer permutes the result back for its output projection. With
    this patch, whenever the active device registers the three "*_strided" kernels (limn_b200.install() does) and the
    call qualifies (4-D float16 / bfloat16 operands of equal batch dims, head dim 64 or 128, no key mask, every
    operand either realised or an unmasked view with contiguous columns whose strides and offset are multiples of
    8 elements), the CUSTOM nodes take the buffers under the views and the views' strides as parameters:

        custom("sdpa_strided", (buffers under q, k, v), (causal, scale, extents, strides))      -> O, L
        custom("sdpa_bwd_q_fused_strided", (..., O, buffer under dO, L), ...)                   -> dQ, delta
        custom("sdpa_bwd_kv_strided", (..., buffer under dO, L, delta), ...)                    -> dK, dV

    O, dQ, dK and dV are written token-major, (batch, t, heads, hd), and returned as permuted views of that, so the
    layer's own `permute(0, 2, 1, 3).reshape(batch, t, heads * hd)` lands on dense memory and costs nothing either.
    Every other call goes to limn's own `Tensor.attention`. Returns a function that undoes the patch."""
    import weakref

    import limn.tensor as frontend
    from limn.ops import Node, Op, accumulate_in, bfloat16, custom, float16
    from limn.schedule import CUT_OPS
    from limn.view import View

    Tensor = frontend.Tensor
    original = Tensor.attention
    if getattr(original, "_limn_b200_views", False):
        return lambda: None

    def under(t):
        """(node whose buffer the kernel reads, (offset, batch, head, row strides) in elements), or None."""
        if t.ndim != 4:
            return None
        if t.node.op is Op.VIEW:
            base, view = t.node.srcs[0], t.node.arg
        else:
            base, view = t.node, View.contiguous(t.shape)
        if view.mask is not None or (view.shape[3] > 1 and view.strides[3] != 1):
            return None
        if view.offset % 8 or any(s % 8 or s < 0 for s in view.strides[:3]) or (view.shape[2] > 1 and view.strides[2] == 0):
            return None
        if base.op is not Op.BUFFER and base.op not in CUT_OPS:
            # an expression: the scheduler would realise it for the view anyway (limn/schedule.py: "an addressed
            # src"); say so once, so that every view over it (q, k and v; forward and backward) shares the buffer.
            # The expression only holds a weak reference to its stand-in: no cycle keeps a buffer alive.
            known = getattr(base, "_limn_b200_realised", None)
            stand_in = known() if known is not None else None
            if stand_in is None:
                stand_in = Node(Op.CONTIGUOUS, (base,), base.dtype, base.shape)
                base._limn_b200_realised = weakref.ref(stand_in)
            base = stand_in
        return base, (view.offset, view.strides[0], view.strides[1], max(view.strides[2], 8))

    def attention(self, k, v, *, causal=False, key_mask=None):
        q = self
        active = frontend.device.active()
        plain = lambda: original(q, k, v, causal=causal, key_mask=key_mask)
        if key_mask is not None or not all(active.has_custom(name) for name in STRIDED_NAMES):
            return plain()
        if not (isinstance(k, Tensor) and isinstance(v, Tensor)) or q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
            return plain()
        if not (q.dtype is k.dtype is v.dtype) or q.dtype not in (float16, bfloat16):
            return plain()
        batch, heads, t_q, hd = q.shape
        t_k = k.shape[2]
        if k.shape != (batch, heads, t_k, hd) or v.shape != (batch, heads, t_k, hd) or hd % 8 or hd > 128 or (causal and t_q != t_k):
            return plain()
        found = [under(t) for t in (q, k, v)]
        if any(f is None for f in found):
            return plain()
        (bq, gq), (bk, gk), (bv, gv) = found
        scale = hd**-0.5
        extents = (batch, heads, t_q, t_k, hd)
        dtype = q.dtype
        rows = (batch, heads, t_q, 1)
        out_node, lse_node = custom(SDPA_STRIDED, (bq, bk, bv), (causal, scale, extents, (gq, gk, gv)),
                                    ((dtype, (batch, t_q, heads, hd)), (accumulate_in(dtype), rows)))
        held = Tensor.from_node(out_node, (q, k, v))
        if held.requires_grad:
            saved_out, saved_lse = Tensor.from_node(out_node), Tensor.from_node(lse_node)
            limns_own = frontend._attention_backward(saved_out.permute(0, 2, 1, 3), saved_lse, q, k, v, None, causal=causal, scale=scale)

            def backward(g):
                """g is the gradient of the token-major O, (batch, t, heads, hd), usually a view of the output
                projection's input gradient."""
                now = frontend.device.active()
                geometry = under(g.permute(0, 2, 1, 3)) if g.ndim == 4 else None
                if frontend.grad_enabled or geometry is None or not all(now.has_custom(name) for name in STRIDED_NAMES[1:]):
                    return limns_own(g.permute(0, 2, 1, 3))
                bg, gg = geometry
                params = (causal, scale, extents, (gq, gk, gv, gg))
                dq, delta = custom(SDPA_BWD_Q_FUSED_STRIDED, (bq, bk, bv, saved_out.node, bg, saved_lse.node), params,
                                   ((dtype, (batch, t_q, heads, hd)), (saved_lse.dtype, rows)))
                dk, dv = custom(SDPA_BWD_KV_STRIDED, (bq, bk, bv, bg, saved_lse.node, delta), params,
                                ((dtype, (batch, t_k, heads, hd)), (dtype, (batch, t_k, heads, hd))))
                return tuple(Tensor.from_node(n).permute(0, 2, 1, 3) for n in (dq, dk, dv))

            held.grad_fn = backward
        return held.permute(0, 2, 1, 3)

    attention._limn_b200_views = True  # type: ignore[attr-defined]
    Tensor.attention = attention

    def undo() -> None:
        Tensor.attention = original

    return undo
