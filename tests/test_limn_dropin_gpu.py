"""limn itself on the GPU with limn_b200's kernels in its CUSTOM registry.

These tests drive limn's own cuda device (driver-API primary context, pooled cuMemAlloc buffers,
launches on the NULL stream, one cuCtxSynchronize per batch, capture replay against new buffers:
limn/backend_cuda.py:272-415, limn/capture.py:152-168) after `limn_b200.install(device)`, and
compare with limn's numpy device, which is the reference for every CUSTOM op
(limn/device.py:160-167). They mirror limn's cuda acceptance tests (tests/test_attention.py:243-396
of the reference) at its shapes and tolerances, add the shapes the tensor-core kernels serve, and
finally run limn's test files themselves, unmodified, with the builders installed by a plugin.

limn is taken from baseline/_ref, the untouched copy `__graft_entry__.build()` stages (or from a
checkout named by LIMN_REFERENCE); without one every test here is skipped, saying so.
"""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
CANDIDATES = [Path(p) for p in (os.environ.get("LIMN_REFERENCE", ""),) if p] + [ROOT / "baseline" / "_ref"]
LIMN = next((p for p in CANDIDATES if (p / "limn" / "backend_cuda.py").is_file()), None)

pytestmark = [
    pytest.mark.gpu,
    pytest.mark.skipif(LIMN is None, reason="limn is not staged under baseline/_ref (run __graft_entry__.build() where the reference is)"),
]

rng = np.random.default_rng(11)


@pytest.fixture(scope="module")
def limn():
    sys.path.insert(0, str(LIMN))
    import limn as package
    import limn.device  # noqa: F401  (so that package.device is there for the tests)

    package.device.set_device("numpy")
    yield package
    package.device.set_device("numpy")
    sys.path.remove(str(LIMN))


@pytest.fixture(scope="module")
def cudev(limn):
    """limn's own CudaDevice with our three builders written over its NVRTC ones, each wrapped to count."""
    from limn import backend_cuda

    import limn_b200

    reason = backend_cuda.cuda_unavailable()
    if reason is not None:
        pytest.fail(f"limn's cuda device cannot run here: {reason}")
    dev = backend_cuda.CudaDevice()
    limn_b200.install(dev)
    dev.b200_counts = {name: {"built": 0, "ran": 0} for name in limn_b200.NAMES}
    for name in limn_b200.NAMES:
        build = dev.custom[name]

        def counted(node, build=build, name=name):
            dev.b200_counts[name]["built"] += 1
            run = build(node)

            def counted_run(inputs, outs):
                dev.b200_counts[name]["ran"] += 1
                run(inputs, outs)

            return counted_run

        dev.custom[name] = counted
    return dev


def read(dev, buf, t) -> np.ndarray:
    from limn.device import NUMPY_DTYPES

    return dev.copyout(buf).view(NUMPY_DTYPES[t.dtype]).reshape(t.shape)


def check(dev, t, tol: float) -> None:
    """One tensor realized on limn's cuda device, then on its numpy device (the reference's own
    check, tests/conftest.py:52-69: device under test first, halves compared as float32)."""
    from limn.ops import HALF_FLOATS

    got = read(dev, dev.execute([t.node])[0], t)
    expected = t.numpy()
    if t.dtype in HALF_FLOATS:
        got, expected = got.astype(np.float32), expected.astype(np.float32)
    np.testing.assert_allclose(got, expected, rtol=tol, atol=tol)


def tensors(limn, dtype_name, q_shape, k_shape, v_shape, scale=1.0):
    dtype = getattr(limn, dtype_name)
    data = [rng.standard_normal(s).astype(np.float32) * scale for s in (q_shape, k_shape, v_shape)]
    return [limn.Tensor(d, dtype=dtype, requires_grad=True) for d in data]


def weighted_grads(limn, dtype_name, q_shape, k_shape, v_shape, causal, key_mask=None):
    q, k, v = tensors(limn, dtype_name, q_shape, k_shape, v_shape)
    out_shape = np.broadcast_shapes(q_shape[:-2], k_shape[:-2], v_shape[:-2]) + (q_shape[-2], v_shape[-1])
    weight = limn.Tensor(rng.standard_normal(out_shape).astype(np.float32), dtype=getattr(limn, dtype_name))
    out = q.attention(k, v, causal=causal, key_mask=key_mask)
    return out, limn.grad((out * weight).sum(), [q, k, v])


# dtype, forward tolerance, backward tolerance: the reference's own (tests/test_attention.py:250-255, :303-308)
TOLERANCES = [("float32", 1e-5, 1e-4), ("float16", 2e-3, 4e-3), ("bfloat16", 1e-2, 3e-2)]

# the reference's shapes (general kernels here: head dims 16 / 24) and the shapes the tcgen05 kernels take
REFERENCE_SHAPES = [((2, 3, 64, 16), (2, 3, 64, 16), (2, 3, 64, 24))]
TENSOR_CORE_SHAPES = [
    ((2, 2, 256, 64), (2, 2, 256, 64), (2, 2, 256, 64)),
    ((1, 2, 384, 128), (1, 2, 384, 128), (1, 2, 384, 128)),
    ((3, 200, 64), (3, 200, 64), (3, 200, 64)),  # ragged: one full tile and a tail
]


@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
@pytest.mark.parametrize("dtype,fwd_tol,bwd_tol", TOLERANCES, ids=[t[0] for t in TOLERANCES])
def test_forward_and_backward_match_limns_numpy_device(limn, cudev, dtype, fwd_tol, bwd_tol, causal):
    shapes = REFERENCE_SHAPES + (TENSOR_CORE_SHAPES if dtype != "float32" else [((2, 2, 256, 64),) * 3])
    before = {name: dict(c) for name, c in cudev.b200_counts.items()}
    for q_shape, k_shape, v_shape in shapes:
        out, grads = weighted_grads(limn, dtype, q_shape, k_shape, v_shape, causal)
        check(cudev, out, fwd_tol)
        for g in grads:
            check(cudev, g, bwd_tol)
    for name, counts in cudev.b200_counts.items():
        assert counts["ran"] > before[name]["ran"], f"{name} never reached a limn_b200 Runner"


@pytest.mark.parametrize(
    "q_shape,k_shape,v_shape,causal",
    [
        ((2, 2, 100, 16), (2, 2, 100, 16), (2, 2, 100, 24), True),
        ((300, 16), (300, 16), (300, 24), True),
        ((40, 8), (72, 8), (72, 12), False),
        ((2, 130, 64), (2, 300, 64), (2, 300, 64), False),  # rectangular on the tensor-core kernels (as float16 below)
    ],
    ids=["ragged causal", "several chunks", "rectangular", "rectangular d64"],
)
def test_ragged_and_rectangular_shapes(limn, cudev, q_shape, k_shape, v_shape, causal):
    """tests/test_attention.py:311-341 of the reference, plus a rectangular case at head dim 64."""
    half = q_shape[-1] == 64
    _, grads = weighted_grads(limn, "float16" if half else "float32", q_shape, k_shape, v_shape, causal)
    for g in grads:
        check(cudev, g, 4e-3 if half else 1e-4)


@pytest.mark.parametrize(
    "dtype,q_shape,k_shape,causal,tol",
    [
        ("float32", (2, 100, 16), (2, 100, 16), True, 1e-4),
        ("float32", (4, 1, 32), (4, 96, 32), False, 1e-4),
        ("bfloat16", (2, 200, 64), (2, 200, 64), True, 3e-2),
        ("float16", (4, 1, 64), (4, 96, 64), False, 4e-3),  # one query row against a partly filled cache, tensor-core kernels
    ],
    ids=["ragged causal f32", "decode row f32", "ragged causal bf16 d64", "decode row f16 d64"],
)
def test_key_mask(limn, cudev, dtype, q_shape, k_shape, causal, tol):
    """tests/test_attention.py:385-396 of the reference: a padded batch and the decode step of a kv cache."""
    live = k_shape[-2] * 2 // 3
    mask = limn.Tensor(np.broadcast_to(np.arange(k_shape[-2]) < live, k_shape[:-1]).astype(np.float32))
    out, grads = weighted_grads(limn, dtype, q_shape, k_shape, k_shape, causal, key_mask=mask)
    check(cudev, out, tol)
    for g in grads:
        check(cudev, g, tol)
    dk = read(cudev, cudev.execute([grads[1].node])[0], grads[1]).astype(np.float32)
    assert np.all(dk[..., live:, :] == 0.0), "hidden keys get exactly-zero gradients"


def test_two_runs_give_the_same_bits(limn, cudev):
    """tests/test_attention.py:258-264, :292-300 of the reference, at a tensor-core shape too."""
    for dtype, shapes in (("float32", REFERENCE_SHAPES[0]), ("bfloat16", TENSOR_CORE_SHAPES[1])):
        out, grads = weighted_grads(limn, dtype, *shapes, True)
        for t in (out, *grads):
            first = cudev.copyout(cudev.execute([t.node])[0])
            second = cudev.copyout(cudev.execute([t.node])[0])
            np.testing.assert_array_equal(first, second)


def test_two_attentions_on_one_input_stay_separate_calls(limn, cudev):
    q, k, v = tensors(limn, "bfloat16", (2, 2, 128, 64), (2, 2, 128, 64), (2, 2, 128, 64))
    check(cudev, q.attention(k, v, causal=True) + q.attention(k, v, causal=True), 2e-2)


def test_the_plan_is_five_calls_with_each_kernel_built_once(limn, cudev):
    """realize(out, dq, dk, dv): sdpa -> (O, L), the copy of dO, the row dot, sdpa_bwd_q, sdpa_bwd_kv; the two
    sibling nodes of each two-output kernel fold into one call (limn/jit.py:213-224)."""
    out, grads = weighted_grads(limn, "bfloat16", (2, 2, 256, 64), (2, 2, 256, 64), (2, 2, 256, 64), True)
    before = {name: dict(c) for name, c in cudev.b200_counts.items()}
    plans_before = set(cudev.plans)
    cudev.execute([out.node] + [g.node for g in grads])
    (key,) = set(cudev.plans) - plans_before
    plan = cudev.plans[key]
    for name in ("sdpa", "sdpa_bwd_q", "sdpa_bwd_kv"):
        assert cudev.b200_counts[name]["built"] - before[name]["built"] == 1, name
        assert cudev.b200_counts[name]["ran"] - before[name]["ran"] == 1, name
    customs = [c for c in plan.calls if len(c.out_nbytes) > 1 or c.fn.__name__ == "counted_run"]
    assert len(customs) == 3
    assert sorted(len(c.out_nbytes) for c in customs) == [1, 2, 2]
    # whatever limn schedules around them (the weighting, the copy of dO, the row dot) is limn's own business;
    # with the upstream gradient handed in as a buffer it is exactly the copy and the reduce
    assert len(plan.calls) >= 5


def test_capture_replays_against_new_buffers(limn, cudev):
    """tests/test_attention.py:353-367 of the reference at a tensor-core shape: two observed calls, then replays
    of the recorded plan with fresh argument and output buffers, all bit-equal to a direct run."""
    import limn_b200

    limn.device.set_device("cuda")
    try:
        limn_b200.install(limn.device.active())  # what a user writes
        data = [rng.standard_normal((2, 2, 256, 64)).astype(np.float32) for _ in range(3)]

        def step(q, k, v):
            return q.attention(k, v, causal=True).realize()

        def fresh():
            return [limn.Tensor(d, dtype=limn.bfloat16) for d in data]

        direct = step(*fresh()).numpy()
        replayed = limn.capture(step)
        for _ in range(4):
            np.testing.assert_array_equal(replayed(*fresh()).numpy(), direct)
    finally:
        limn.device.set_device("numpy")


def test_the_frontend_patch_for_the_fused_row_dot(limn):
    """limn_b200.frontend.fuse_row_dot(): with the cuda device active, limn's autograd then builds
    "sdpa_bwd_q_fused" -> (dQ, delta) in place of its row-dot reduce and "sdpa_bwd_q". The gradients match limn's
    numpy device (whose graph stays limn's own: it has no such kernel) and the unpatched cuda run, and the plan is
    a call shorter."""
    from limn.ops import Op, topological

    import limn_b200
    from limn_b200 import frontend as patch

    shape = (2, 2, 256, 64)
    data = [rng.standard_normal(shape).astype(np.float32) for _ in range(4)]

    def grads_on(device_name: str):
        limn.device.set_device(device_name)
        try:
            dev = limn.device.active()
            if device_name == "cuda":
                limn_b200.install(dev)
            q, k, v = (limn.Tensor(d, dtype=limn.bfloat16, requires_grad=True) for d in data[:3])
            out = q.attention(k, v, causal=True)
            grads = limn.grad((out * limn.Tensor(data[3], dtype=limn.bfloat16)).sum(), [q, k, v])
            names = [n.arg.name for n in topological([g.node for g in grads]) if n.op is Op.CUSTOM]
            calls = None
            if device_name == "cuda":
                limn.realize(*grads)
                calls = max(len(plan.calls) for plan in dev.plans.values())
            return [g.numpy().astype(np.float32) for g in grads], names, calls
        finally:
            limn.device.set_device("numpy")

    want, _, _ = grads_on("numpy")
    plain, plain_names, plain_calls = grads_on("cuda")
    undo = patch.fuse_row_dot()
    try:
        on_numpy, numpy_names, _ = grads_on("numpy")
        fused, fused_names, fused_calls = grads_on("cuda")
    finally:
        undo()
    assert "sdpa_bwd_q_fused" in fused_names and "sdpa_bwd_q" not in fused_names
    assert "sdpa_bwd_q_fused" not in plain_names and "sdpa_bwd_q_fused" not in numpy_names
    assert fused_calls < plain_calls, (fused_calls, plain_calls)
    for got in (plain, fused, on_numpy):
        for g, w in zip(got, want, strict=True):
            np.testing.assert_allclose(g, w, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("hd", [64, 40], ids=["hd 64", "hd 40 (zero-padded in the 64 kernel)"])
def test_attention_over_views_in_place(limn, hd):
    """limn_b200.frontend.read_views_in_place(): an attention layer as a model writes it (one projection, q, k, v as
    slices of it, the result permuted back for the output projection) on limn's cuda device: the gradient with
    respect to the projection matches limn's numpy device, the plan has no copy kernel per operand any more, and the
    strided Runners are what ran."""
    import limn_b200
    from limn_b200 import frontend as patch

    b, t, heads = 2, 200, 3
    data = rng.standard_normal((b, t, 3 * heads * hd)).astype(np.float32)
    weight = rng.standard_normal((b, t, heads * hd)).astype(np.float32)

    def layer_gradient(device_name: str):
        limn.device.set_device(device_name)
        try:
            dev = limn.device.active()
            ran = []
            if device_name == "cuda":
                limn_b200.install(dev)
                for name in list(dev.custom):
                    build = dev.custom[name]
                    dev.custom[name] = lambda node, build=build, name=name: (ran.append(name), build(node))[1]
            x = limn.Tensor(data, requires_grad=True)
            q, k, v = x.cast(limn.bfloat16).reshape(b, t, 3, heads, hd).permute(2, 0, 3, 1, 4)
            y = q.attention(k, v, causal=True).permute(0, 2, 1, 3).reshape(b, t, heads * hd).cast(limn.float32)
            (g,) = limn.grad((y * limn.Tensor(weight)).sum(), [x])
            calls = None
            if device_name == "cuda":
                limn.realize(y, g)
                calls = max(len(plan.calls) for plan in dev.plans.values())
            return y.numpy(), g.numpy(), calls, ran
        finally:
            limn.device.set_device("numpy")

    want_y, want_g, _, _ = layer_gradient("numpy")
    plain_y, plain_g, plain_calls, plain_ran = layer_gradient("cuda")
    undo = patch.read_views_in_place()
    try:
        got_y, got_g, got_calls, got_ran = layer_gradient("cuda")
    finally:
        undo()
    assert set(got_ran) == {"sdpa_strided", "sdpa_bwd_q_fused_strided", "sdpa_bwd_kv_strided"}, got_ran
    assert set(plain_ran) == {"sdpa", "sdpa_bwd_q", "sdpa_bwd_kv"}, plain_ran
    assert got_calls <= plain_calls - 4, (got_calls, plain_calls)  # three operand copies, the dO copy, the row dot ...
    for got, want in ((plain_y, want_y), (got_y, want_y)):
        np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2)
    for got, want in ((plain_g, want_g), (got_g, want_g)):
        np.testing.assert_allclose(got, want, rtol=3e-2, atol=3e-2)


def test_a_gpt_training_step_under_capture(limn):
    """The caller of the GPT attention layer: a two-layer byte-level GPT step shaped like limn's
    examples/train_stories.py (its model and step, :26-56 and :140-147 there) with bfloat16 attention operands,
    captured and replayed on limn's cuda device with our kernels installed, against the same step on limn's numpy
    device from the same seed. Synthetic tokens stand in for the TinyStories text the example downloads."""
    import bench

    import limn_b200

    tokens = np.random.default_rng(5).integers(0, 256, size=(2, 129)).astype(np.int32)
    ran = {"sdpa": 0, "sdpa_bwd_q": 0, "sdpa_bwd_kv": 0}

    def losses(device_name: str, install: bool) -> list[float]:
        limn.device.set_device(device_name)
        try:
            if install:
                dev = limn_b200.install(limn.device.active())
                for name in ran:
                    build = dev.custom[name]

                    def counted(node, build=build, name=name):
                        run = build(node)

                        def counted_run(inputs, outs):
                            ran[name] += 1
                            run(inputs, outs)

                        return counted_run

                    dev.custom[name] = counted
            limn.set_seed(0)
            step, _ = bench.gpt_step(limn, dim=128, heads=2, layers=2, ctx=128, attention_dtype=limn.bfloat16)
            replayed = limn.capture(step)
            return [replayed(limn.Tensor(tokens[:, :-1]), limn.Tensor(tokens[:, 1:])).item() for _ in range(4)]
        finally:
            limn.device.set_device("numpy")

    want = losses("numpy", False)
    got = losses("cuda", True)
    assert all(count >= 2 * 4 for count in ran.values()), ran  # two layers, four steps (two observed, two replayed)
    np.testing.assert_allclose(got, want, rtol=5e-3)
    assert got[-1] < got[0]


def test_limns_own_test_files_pass_with_the_builders_installed(tmp_path):
    """limn's tests/test_attention.py and tests/test_jit.py, byte for byte as the reference has them, in a
    process of their own with tests/limn_dropin_plugin.py installing the builders on every CudaDevice."""
    report = tmp_path / "dropin.json"
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([str(LIMN), str(ROOT), str(ROOT / "tests")] + ([env["PYTHONPATH"]] if env.get("PYTHONPATH") else []))
    env["LIMN_B200_DROPIN_REPORT"] = str(report)
    env["PYTHONDONTWRITEBYTECODE"] = "1"
    done = subprocess.run(
        [sys.executable, "-m", "pytest", "-p", "limn_dropin_plugin", "-p", "no:cacheprovider", "-q", "-rs",
         "tests/test_attention.py", "tests/test_jit.py"],
        cwd=LIMN, env=env, capture_output=True, text=True, timeout=1500,
    )
    tail = "\n".join(done.stdout.splitlines()[-25:])
    print(tail)
    assert done.returncode == 0, f"limn's tests failed with limn_b200 installed:\n{tail}\n{done.stderr[-2000:]}"
    counts = json.loads(report.read_text())["counts"]
    for name in ("sdpa", "sdpa_bwd_q", "sdpa_bwd_kv"):
        assert counts[name]["ran"] > 0, f"limn's tests never reached the limn_b200 Runner for {name}: {counts}"
    assert "skipped" not in done.stdout.splitlines()[-1] or "no CUDA" not in done.stdout, "the cuda tests were skipped"
    keep = os.environ.get("LIMN_B200_TEST_REPORTS")  # a directory in which to leave the summary, if the caller wants it
    if keep and Path(keep).is_dir():
        (Path(keep) / "limn_reference_tests.txt").write_text(tail + "\n" + json.dumps(counts) + "\n")
