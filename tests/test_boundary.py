"""The drop-in boundary without a GPU: the library loads and exports every symbol the header
declares, argument checks answer before any CUDA call, and the registry builders read nodes
the way limn's own cuda device does."""

from __future__ import annotations

import os
import re
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
# limn itself, where it is at hand: the copy __graft_entry__.build() stages, or a checkout named by LIMN_REFERENCE
REFERENCE = next((p for p in (Path(os.environ.get("LIMN_REFERENCE", "")), ROOT / "baseline" / "_ref") if (p / "limn" / "sdpa.py").is_file()),
                 ROOT / "baseline" / "_ref")


def declared_functions() -> list[str]:
    text = (ROOT / "include" / "limn_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"\b(limn_b200_[a-z0-9_]+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    from limn_b200._lib import SIGNATURES, lib

    names = declared_functions()
    assert len(names) >= 25 and len(set(names)) == len(names)
    loaded = lib()
    for name in names:
        assert hasattr(loaded, name), f"{name} is declared in include/limn_b200.h but not exported"
    assert set(names) == set(SIGNATURES), "the ctypes table and the header disagree"
    assert loaded.limn_b200_version() >= 100


def test_argument_checks_answer_without_a_device():
    from limn_b200._lib import lib

    fwd = lib().limn_b200_sdpa_fwd
    err = lambda: lib().limn_b200_last_error().decode()
    one = 1  # any non-null pointer value; the checks below fail before anything is dereferenced
    assert fwd(one, one, one, None, one, one, 9, 1, 4, 4, 8, 8, 0, 1.0, None) == 1 and "dtype" in err()
    assert fwd(one, one, one, None, one, one, 0, 1, 4, 5, 8, 8, 1, 1.0, None) == 1 and "square keys" in err()
    assert fwd(one, one, one, None, one, one, 0, 1, 0, 4, 8, 8, 0, 1.0, None) == 1 and "positive" in err()
    assert fwd(None, one, one, None, one, one, 0, 1, 4, 4, 8, 8, 0, 1.0, None) == 1 and "null" in err()
    assert lib().limn_b200_sdpa_bwd_q(one, one, one, one, one, None, None, one, 0, 1, 4, 4, 8, 8, 0, 1.0, None) == 1
    assert lib().limn_b200_sdpa_bwd_kv(one, one, one, one, one, one, None, one, None, 0, 1, 4, 4, 8, 8, 0, 1.0, None) == 1
    # an empty batch is a successful no-op
    assert fwd(one, one, one, None, one, one, 0, 0, 4, 4, 8, 8, 0, 1.0, None) == 0 and err() == ""
    # the layout entry points check their own arguments first, then the same ones
    laid = lib().limn_b200_sdpa_fwd_layout
    assert laid(one, one, one, None, one, one, 7, 2, 1, 2, 4, 4, 64, 64, 0, 1.0, None) == 1 and "layout" in err()
    assert laid(one, one, one, None, one, one, 1, 2, 1, 0, 4, 4, 64, 64, 0, 1.0, None) == 1 and "heads" in err()
    assert laid(one, one, one, None, one, one, 1, 2, 1, 2, 4, 5, 64, 64, 1, 1.0, None) == 1 and "square keys" in err()
    assert laid(one, one, one, None, one, one, 1, 2, 0, 2, 4, 4, 64, 64, 0, 1.0, None) == 0 and err() == ""
    assert lib().limn_b200_sdpa_delta_layout(one, one, one, 5, 2, 1, 2, 4, 64, None) == 1 and "layout" in err()


def test_nccl_entry_points_fail_with_codes_not_aborts(monkeypatch):
    """The sharded path's failure handling, host side only: misuse and a communication library that cannot be
    loaded come back as status codes with a message."""
    import ctypes

    from limn_b200._lib import BAD_ARGUMENT, UNSUPPORTED, last_error, lib

    L = lib()
    buf = ctypes.create_string_buffer(128)
    assert L.limn_b200_nccl_init(2, 2, buf) == BAD_ARGUMENT and "not one of 2 ranks" in last_error()
    assert L.limn_b200_nccl_init(0, 2, None) == BAD_ARGUMENT
    assert L.limn_b200_nccl_all_gather(1, 1, 16, None) == BAD_ARGUMENT and "no communicator" in last_error()
    assert L.limn_b200_nccl_unique_id(None) == BAD_ARGUMENT
    assert L.limn_b200_nccl_destroy() == 0  # nothing to destroy is not an error


def test_a_missing_nccl_is_reported(tmp_path):
    """In a process of its own (the library is loaded once per process): a named NCCL that does not exist."""
    import subprocess

    code = ("import ctypes, sys; sys.path.insert(0, %r); from limn_b200._lib import lib, last_error; "
            "rc = lib().limn_b200_nccl_unique_id(ctypes.create_string_buffer(128)); print(rc, last_error())") % str(ROOT)
    done = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, LIMN_B200_NCCL_LIBRARY=str(tmp_path / "libnccl.so.2")),
                          capture_output=True, text=True, timeout=120)
    assert done.returncode == 0, done.stderr
    assert done.stdout.startswith("2 nccl: cannot load"), done.stdout


def test_dispatch_policy():
    from limn_b200._lib import PATH_GENERAL, PATH_TCGEN05, lib

    path = lib().limn_b200_sdpa_path
    # dtype codes: f32 0, f16 1, bf16 2, f64 3
    assert path(2, 256, 4096, 4096, 128, 128, 1, 0, 128**-0.5) == PATH_TCGEN05
    assert path(1, 256, 2048, 2048, 64, 64, 0, 0, 0.125) == PATH_TCGEN05
    assert path(2, 1, 1, 300, 64, 64, 0, 0, 0.125) == 2  # PATH_DECODE: one query row against many keys
    assert path(2, 2, 64, 64, 64, 64, 0, 1, 0.125) == PATH_TCGEN05  # key mask, 16-bit storage
    assert path(2, 2, 64, 64, 32, 32, 1, 0, 0.2) == PATH_TCGEN05  # a narrower head runs zero-padded in the 64 kernel
    assert path(1, 2, 64, 64, 96, 96, 0, 0, 0.1) == PATH_TCGEN05  # or in the 128 kernel
    assert path(2, 2, 64, 64, 64, 128, 0, 0, 0.125) == PATH_TCGEN05  # hd != hd_v: each operand at its own width
    for general in (
        (0, 2, 128, 128, 32, 32, 1, 0, 32**-0.5),  # float32 computes at its own width
        (3, 2, 64, 64, 64, 64, 1, 0, 0.125),  # float64
        (2, 2, 64, 64, 36, 36, 1, 0, 0.2),  # a head dim that is no multiple of 8
        (2, 2, 64, 64, 136, 136, 1, 0, 0.2),  # or above 128
        (2, 2, 64, 64, 64, 132, 0, 0, 0.125),  # hd_v no multiple of 8
        (2, 2, 64, 64, 64, 64, 0, 0, -0.125),  # non-positive scale
    ):
        assert path(*general) == PATH_GENERAL
    assert path(2, 2, 64, 65, 64, 64, 1, 0, 0.125) == -1


def _nodes(host, dtype, qs, ks, vs, causal, mask=False):
    q, k, v = (host.Node((), dtype, s) for s in (qs, ks, vs))
    tail = (host.Node((), dtype, qs[:-2] + ks[-2:-1]),) if mask else ()
    outs = ((dtype, qs[:-1] + vs[-1:]), (host.accumulate_in(dtype), qs[:-1] + (1,)))
    return host.custom("sdpa", (q, k, v) + tail, (causal, qs[-1] ** -0.5), outs)


def test_builders_read_a_node_like_the_reference_does():
    import limn_standin as host
    from limn_b200 import registry

    out, lse = _nodes(host, host.bfloat16, (2, 3, 100, 64), (2, 3, 100, 64), (2, 3, 100, 64), True)
    assert out.arg.index == 0 and lse.arg.index == 1 and out.srcs is lse.srcs
    form = registry.Form(out, 3)
    assert (form.bh, form.t_q, form.t_k, form.hd, form.hd_v, form.causal, form.has_mask) == (6, 100, 100, 64, 64, True, False)
    assert form.dtype == 2 and form.outputs == 2
    masked = _nodes(host, host.float32, (40, 8), (72, 8), (72, 12), False, mask=True)[0]
    form = registry.Form(masked, 3)
    assert (form.bh, form.t_q, form.t_k, form.hd, form.hd_v, form.has_mask) == (1, 40, 72, 8, 12, True)
    for name in registry.NAMES:
        assert callable(registry.BUILDERS[name])
    run = registry.build_sdpa(out)
    with pytest.raises(RuntimeError, match="built for 3 inputs and 2 outputs"):
        run([], [])


def test_builders_refuse_what_the_ops_cannot_be():
    import limn_standin as host
    from limn_b200 import registry

    with pytest.raises(ValueError, match="square keys"):
        registry.build_sdpa(_nodes(host, host.float32, (4, 8), (5, 8), (5, 8), True)[0])
    with pytest.raises(ValueError, match="head dims differ"):
        registry.build_sdpa(_nodes(host, host.float32, (4, 8), (4, 6), (4, 8), False)[0])
    int8 = host.DType("int8", 1)
    with pytest.raises(NotImplementedError, match="int8"):
        registry.build_sdpa(_nodes(host, int8, (4, 8), (4, 8), (4, 8), False)[0])


def test_install_needs_a_registry():
    import limn_b200

    class Bare:
        pass

    with pytest.raises(TypeError, match="no CUSTOM registry"):
        limn_b200.install(Bare())

    class WithRegistry:
        def __init__(self):
            self.custom = {}

    dev = limn_b200.install(WithRegistry())
    assert set(dev.custom) == {"sdpa", "sdpa_bwd_q", "sdpa_bwd_kv", "sdpa_bwd_q_fused", "sdpa_strided", "sdpa_bwd_q_fused_strided",
                               "sdpa_bwd_kv_strided"}


def test_installed_finish_reports_a_kernel_that_gave_up(monkeypatch):
    """install() wraps finish(): with a status word set (a fake library here, no GPU), the batch barrier raises
    the RuntimeError limn raises for a failed kernel (limn/backend_cuda.py:154-162, :349); a batch without one of
    our launches does not even read the word."""
    import limn_b200
    from limn_b200 import registry

    reads = []

    class FakeLibrary:
        word = 0x57410203

        def limn_b200_device_status(self, ref):
            reads.append(self.word)
            ref._obj.value, code = self.word, (4 if self.word else 0)
            self.word = 0
            return code

        def limn_b200_last_error(self):
            return b"a kernel gave up"

    class Device:
        def __init__(self):
            self.custom, self.barriers = {}, 0

        def finish(self):
            self.barriers += 1

    dev = limn_b200.install(Device())
    limn_b200.install(dev)  # installing twice wraps once
    fake = FakeLibrary()
    monkeypatch.setattr(registry, "lib", lambda: fake)
    monkeypatch.setattr(registry, "_launched_since_check", False)
    dev.finish()
    assert reads == [] and dev.barriers == 1
    registry._note_launch()
    with pytest.raises(RuntimeError, match=r"cuda: waiting for the batch: .*status 0x57410203"):
        dev.finish()
    registry._note_launch()
    dev.finish()  # the word was cleared by the read
    assert reads == [0x57410203, 0] and dev.barriers == 3


def test_host_validation_matches_the_frontend_messages():
    import limn_standin as host

    z = lambda *s: np.zeros(s, np.float32)
    with pytest.raises(ValueError, match="2D\\+ tensors"):
        host._validate(z(8), z(8), z(8), None, False)
    with pytest.raises(ValueError, match="key counts differ"):
        host._validate(z(4, 8), z(5, 8), z(6, 8), None, False)
    with pytest.raises(ValueError, match="one flag per key"):
        host._validate(z(4, 8), z(5, 8), z(5, 8), z(4), False)


@pytest.mark.skipif(not (REFERENCE / "limn").is_dir(), reason="the reference checkout is not on this machine")
def test_install_into_limns_own_registry_and_plan():
    """With limn importable: install() on one of its CompiledDevices, then let its frontend,
    scheduler and plan builder reach our builders with real nodes (nothing is launched)."""
    sys.path.insert(0, str(REFERENCE))
    try:
        import limn
        from limn import backend_c
        from limn.ops import Op, topological
        from limn.tensor import Tensor

        import limn_b200
        from limn_b200 import registry

        dev = limn_b200.install(backend_c.CDevice())
        assert all(dev.has_custom(name) for name in registry.NAMES)
        seen = []
        for name in registry.NAMES:
            build = dev.custom[name]
            dev.custom[name] = lambda node, build=build: (seen.append(registry.Form(node, 3 if node.arg.name == "sdpa" else 6)), build(node))[1]
        import limn.device as device_module

        original = device_module.DEVICES["c"]
        device_module.DEVICES["c"] = lambda: dev  # the device set_device("c") hands out
        limn.set_device("c")
        rng = np.random.default_rng(0)
        q, k, v = (Tensor(rng.standard_normal((2, 3, 64, 16)).astype(np.float32), requires_grad=True) for _ in range(3))
        out = q.attention(k, v, causal=True)
        grads = limn.grad((out * out).sum(), [q, k, v])
        nodes = topological([g.node for g in grads])
        customs = [n for n in nodes if n.op is Op.CUSTOM]
        assert {n.arg.name for n in customs} == set(registry.NAMES)
        plan = dev.plan_of(nodes, {n: i for i, n in enumerate(nodes)}, [g.node for g in grads]) if hasattr(dev, "plan_of") else None
        assert plan is not None
        assert sorted(f.name for f in seen) == sorted(registry.NAMES), "each kernel is built once per plan (sibling merge)"
        by_name = {f.name: f for f in seen}
        assert (by_name["sdpa"].bh, by_name["sdpa"].t_q, by_name["sdpa"].hd, by_name["sdpa"].outputs) == (6, 64, 16, 2)
        assert by_name["sdpa_bwd_kv"].outputs == 2 and by_name["sdpa_bwd_q"].inputs == 6
    finally:
        sys.path.remove(str(REFERENCE))
        import limn.device as device_module

        device_module.set_device("numpy")
        if "original" in locals():
            device_module.DEVICES["c"] = original


@pytest.mark.skipif(not (REFERENCE / "limn").is_dir(), reason="the reference checkout is not on this machine")
def test_the_frontend_patch_swaps_the_row_dot_for_the_fused_op():
    """limn_b200.frontend.fuse_row_dot(): on a device with "sdpa_bwd_q_fused" the backward graph holds the fused
    node (dQ, delta) feeding "sdpa_bwd_kv" and no row-dot reduce; on limn's numpy device, which has no such
    kernel, the graph is limn's own; undo() restores limn's function. Graph level only, nothing is launched."""
    sys.path.insert(0, str(REFERENCE))
    try:
        import limn
        import limn.device as device_module
        import limn.tensor as frontend
        from limn import backend_c
        from limn.ops import Op, topological

        import limn_b200
        from limn_b200 import frontend as patch

        def backward_nodes():
            rng = np.random.default_rng(0)
            q, k, v = (limn.Tensor(rng.standard_normal((2, 3, 64, 16)).astype(np.float32), requires_grad=True) for _ in range(3))
            out = q.attention(k, v, causal=True)
            grads = limn.grad((out * out).sum(), [q, k, v])
            return topological([g.node for g in grads])

        before = frontend._attention_backward
        undo = patch.fuse_row_dot()
        try:
            assert patch.fuse_row_dot() is not None  # patching twice is harmless
            names = [n.arg.name for n in backward_nodes() if n.op is Op.CUSTOM]  # numpy device: limn's own graph
            assert "sdpa_bwd_q_fused" not in names and "sdpa_bwd_q" in names
            dev = limn_b200.install(backend_c.CDevice())
            original = device_module.DEVICES["c"]
            device_module.DEVICES["c"] = lambda: dev
            try:
                limn.set_device("c")
                nodes = backward_nodes()
            finally:
                device_module.DEVICES["c"] = original
                limn.set_device("numpy")
            customs = [n for n in nodes if n.op is Op.CUSTOM]
            assert {n.arg.name for n in customs} == {"sdpa", "sdpa_bwd_q_fused", "sdpa_bwd_kv"}
            fused = [n for n in customs if n.arg.name == "sdpa_bwd_q_fused"]
            assert sorted(n.arg.index for n in fused) == [0, 1] and len(fused[0].srcs) == 6
            kv = next(n for n in customs if n.arg.name == "sdpa_bwd_kv")
            assert kv.srcs[5] in fused and kv.srcs[5].arg.index == 1, "the dK/dV op reads the delta the fused op wrote"
            assert not any(n.op is Op.SUM and n.shape[-1] == 1 and len(n.shape) == 4 for n in nodes), "the row-dot reduce is gone"
        finally:
            undo()
        assert frontend._attention_backward is before
    finally:
        sys.path.remove(str(REFERENCE))


@pytest.mark.skipif(not (REFERENCE / "limn").is_dir(), reason="the reference checkout is not on this machine")
def test_the_frontend_patch_hands_views_over_in_place():
    """limn_b200.frontend.read_views_in_place(): q, k, v taken as slices of one projection reach the CUSTOM nodes
    as the buffer under them plus strides (no CONTIGUOUS copy per operand), the result comes back token-major, and
    calls that do not qualify (float32 here) go to limn's own Tensor.attention. Graph level only."""
    sys.path.insert(0, str(REFERENCE))
    try:
        import limn
        import limn.device as device_module
        from limn import backend_c
        from limn.ops import Op, topological

        import limn_b200
        from limn_b200 import frontend as patch

        undo = patch.read_views_in_place()
        dev = limn_b200.install(backend_c.CDevice())
        original = device_module.DEVICES["c"]
        device_module.DEVICES["c"] = lambda: dev
        try:
            limn.set_device("c")
            b, t, heads, hd = 2, 16, 2, 64
            rng = np.random.default_rng(0)

            def layer_gradient(dtype):
                x = limn.Tensor(rng.standard_normal((b, t, 3 * heads * hd)).astype(np.float32), requires_grad=True)
                q, k, v = x.cast(dtype).reshape(b, t, 3, heads, hd).permute(2, 0, 3, 1, 4)
                y = q.attention(k, v, causal=True).permute(0, 2, 1, 3).reshape(b, t, heads * hd).cast(limn.float32)
                (g,) = limn.grad((y * y).sum(), [x])
                return topological([g.node])

            nodes = layer_gradient(limn.bfloat16)
            customs = [n for n in nodes if n.op is Op.CUSTOM and n.arg.index == 0]
            assert sorted(n.arg.name for n in customs) == ["sdpa_bwd_kv_strided", "sdpa_bwd_q_fused_strided", "sdpa_strided"]
            forward = next(n for n in customs if n.arg.name == "sdpa_strided")
            causal, scale, extents, views = forward.arg.params
            row = 3 * heads * hd
            assert extents == (b, heads, t, t, hd) and causal is True
            assert views == ((0, t * row, hd, row), (heads * hd, t * row, hd, row), (2 * heads * hd, t * row, hd, row))
            assert forward.srcs[0] is forward.srcs[1] is forward.srcs[2], "q, k and v sit on one buffer"
            assert forward.arg.outs[0][1] == (b, t, heads, hd), "the result is token-major"
            # one buffer for the projection, one for the gradient that comes back: no copy per operand
            assert sum(1 for n in nodes if n.op is Op.CONTIGUOUS) <= 3
            dq = next(n for n in customs if n.arg.name == "sdpa_bwd_q_fused_strided")
            assert dq.arg.params[3][3] == (0, t * heads * hd, hd, heads * hd), "dO is read token-major where it lies"
            names = {n.arg.name for n in layer_gradient(limn.float32) if n.op is Op.CUSTOM}
            assert names == {"sdpa", "sdpa_bwd_q", "sdpa_bwd_kv"}, "float32 is not served strided: limn's own path"
        finally:
            device_module.DEVICES["c"] = original
            limn.set_device("numpy")
            undo()
        assert not getattr(limn.Tensor.attention, "_limn_b200_views", False)
    finally:
        sys.path.remove(str(REFERENCE))
