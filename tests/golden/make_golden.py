"""Generate tests/golden/sdpa_golden.npz by running the reference's own numpy kernels.

Run from the repository root in a container that has the reference checked out:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/limn-checkout

It imports limn.sdpa from that checkout, calls the three registry entries
(limn/sdpa.py:209-221, the functions the numpy device dispatches CUSTOM nodes to) on seeded
inputs and stores inputs and outputs. The fixture travels with the repository; the reference
does not have to. bfloat16 arrays are stored as their uint16 bit patterns ("<name>__bf16").
"""

from __future__ import annotations

import os
import sys
from pathlib import Path
from types import SimpleNamespace

import ml_dtypes
import numpy as np

BF16 = np.dtype(ml_dtypes.bfloat16)
HERE = Path(__file__).resolve().parent

# name, dtype, q shape, k shape, v shape, causal, mask kind, (q scale, k scale, v kind), seed
CASES = [
    ("cfg1_f32_causal", "float32", (1, 2, 128, 32), (1, 2, 128, 32), (1, 2, 128, 32), True, None, (1.0, 1.0, "normal"), 0),
    ("bf16_causal_d64", "bfloat16", (1, 2, 256, 64), (1, 2, 256, 64), (1, 2, 256, 64), True, None, (1.0, 1.0, "normal"), 2),
    ("bf16_full_d64", "bfloat16", (2, 1, 256, 64), (2, 1, 256, 64), (2, 1, 256, 64), False, None, (1.0, 1.0, "normal"), 4),
    ("bf16_causal_d128", "bfloat16", (1, 1, 384, 128), (1, 1, 384, 128), (1, 1, 384, 128), True, None, (0.5, 0.5, "half"), 3),
    ("bf16_ragged_sharp_d128", "bfloat16", (1, 2, 200, 128), (1, 2, 200, 128), (1, 2, 200, 128), True, None, (2.0, 2.0, "uniform"), 5),
    ("bf16_full_rect_d128", "bfloat16", (2, 150, 128), (2, 333, 128), (2, 333, 128), False, None, (1.0, 1.0, "normal"), 6),
    ("f16_causal_hd16_hdv24", "float16", (2, 3, 64, 16), (2, 3, 64, 16), (2, 3, 64, 24), True, None, (1.0, 1.0, "normal"), 7),
    ("f64_causal_hdv16", "float64", (2, 64, 32), (2, 64, 32), (2, 64, 16), True, None, (1.0, 1.0, "normal"), 8),
    ("f32_rect_40x72", "float32", (40, 8), (72, 8), (72, 12), False, None, (1.0, 1.0, "normal"), 9),
    ("f32_tail_100", "float32", (2, 2, 100, 16), (2, 2, 100, 16), (2, 2, 100, 24), True, None, (1.0, 1.0, "normal"), 10),
    ("f32_rows_300", "float32", (300, 16), (300, 16), (300, 24), True, None, (1.0, 1.0, "normal"), 11),
    ("f32_mask_holes", "float32", (2, 3, 64, 16), (2, 3, 64, 16), (2, 3, 64, 24), False, "holes", (1.0, 1.0, "normal"), 12),
    ("f32_mask_pad_causal", "float32", (2, 100, 16), (2, 100, 16), (2, 100, 16), True, "pad", (1.0, 1.0, "normal"), 13),
    ("f32_decode_row_mask", "float32", (4, 1, 32), (4, 96, 32), (4, 96, 32), False, "pad", (1.0, 1.0, "normal"), 14),
    ("bf16_mask_holes_d64", "bfloat16", (2, 130, 64), (2, 130, 64), (2, 130, 64), False, "holes", (1.0, 1.0, "normal"), 15),
    ("f32_hot_q", "float32", (128, 64), (128, 64), (128, 64), True, None, (100.0, 1.0, "normal"), 16),
]


def inputs_for(case):
    name, dtype, qs, ks, vs, causal, mask_kind, (q_mul, k_mul, v_kind), seed = case
    dt = BF16 if dtype == "bfloat16" else np.dtype(dtype)
    rng = np.random.default_rng(seed)
    q = (rng.standard_normal(qs) * q_mul).astype(dt)
    k = (rng.standard_normal(ks) * k_mul).astype(dt)
    if v_kind == "uniform":
        v = rng.uniform(-1.0, 1.0, vs).astype(dt)
    elif v_kind == "half":
        v = (rng.standard_normal(vs) * 0.5).astype(dt)
    else:
        v = rng.standard_normal(vs).astype(dt)
    do = rng.standard_normal(qs[:-1] + vs[-1:]).astype(dt)
    mask = None
    if mask_kind == "holes":
        mask = (rng.random(ks[:-1]) > 0.3).astype(dt)
        mask[..., 0] = 1  # no row may lose every key
    elif mask_kind == "pad":
        live = ks[-2] * 2 // 3
        mask = np.broadcast_to((np.arange(ks[-2]) < live), ks[:-1]).astype(dt)
    scale = float(qs[-1]) ** -0.5
    return q, k, v, do, mask, causal, scale


def store(bundle: dict, key: str, array: np.ndarray) -> None:
    if array.dtype == BF16:
        bundle[key + "__bf16"] = array.view(np.uint16)
    else:
        bundle[key] = array


def main() -> None:
    # the reference checkout: an argument, LIMN_REFERENCE, or the copy the build stages under baseline/_ref
    staged = Path(__file__).resolve().parents[2] / "baseline" / "_ref"
    checkout = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LIMN_REFERENCE", str(staged))
    sys.path.insert(0, checkout)
    from limn import sdpa as ref  # the reference's numpy kernels

    bundle: dict[str, np.ndarray] = {}
    for case in CASES:
        name = case[0]
        q, k, v, do, mask, causal, scale = inputs_for(case)
        tail = [] if mask is None else [mask]
        arg = SimpleNamespace(params=(causal, scale))
        out, lse = ref.KERNELS[ref.SDPA]([q, k, v, *tail], arg)
        wide = lse.dtype
        delta = (do.astype(wide) * out.astype(wide)).sum(axis=-1, keepdims=True)  # limn/tensor.py:705-706
        held = [q, k, v, do, lse, delta, *tail]
        (dq,) = ref.KERNELS[ref.SDPA_BWD_Q](held, arg)
        dk, dv = ref.KERNELS[ref.SDPA_BWD_KV](held, arg)
        for key, array in (("out", out), ("lse", lse), ("delta", delta), ("dq", dq), ("dk", dk), ("dv", dv)):
            store(bundle, f"{name}/{key}", np.ascontiguousarray(array))
        print(f"{name:28s} out {out.dtype} {out.shape} lse {lse.dtype}")
    np.savez_compressed(HERE / "sdpa_golden.npz", **bundle)
    print("wrote", HERE / "sdpa_golden.npz", (HERE / "sdpa_golden.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
