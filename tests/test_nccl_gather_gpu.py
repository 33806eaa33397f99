"""A sharded run without torch: two processes, one GPU each, compute their halves of a batch through the C ABI and
gather the outputs with limn_b200_nccl_all_gather; the assembled tensor is compared with the CPU oracle.

Needs two GPUs (skipped with fewer). The ranks are child processes of this test: rank 0 makes the NCCL id and leaves
it in a file, rank 1 picks it up there, which is all the "launcher" a host needs. Every wait in the children is
bounded, and they exit between steps, never with a collective in flight.
"""

from __future__ import annotations

import os
import subprocess
import sys
import time
from pathlib import Path

import ml_dtypes
import numpy as np

BF16 = np.dtype(ml_dtypes.bfloat16)
ROOT = Path(__file__).resolve().parent.parent
BH, T, D = 6, 384, 128


def inputs():
    rng = np.random.default_rng(44)
    return [rng.standard_normal((BH, T, D)).astype(np.float32).astype(BF16) for _ in range(3)]


def rank_main(rank: int, world: int, scratch: Path) -> None:
    sys.path.insert(0, str(ROOT))
    import ctypes

    from limn_b200 import runtime
    from limn_b200._lib import check, lib

    L = lib()
    runtime.set_device(rank)
    id_file = scratch / "nccl_id.bin"
    if rank == 0:
        buf = ctypes.create_string_buffer(128)
        check(L.limn_b200_nccl_unique_id(buf), "making the NCCL id")
        (scratch / "nccl_id.tmp").write_bytes(buf.raw)
        os.replace(scratch / "nccl_id.tmp", id_file)
    deadline = time.time() + 120
    while not id_file.exists():
        if time.time() > deadline:
            raise SystemExit("rank 0 never published the NCCL id")
        time.sleep(0.05)
    check(L.limn_b200_nccl_init(rank, world, id_file.read_bytes()), "joining the communicator")
    per_rank = BH // world
    q, k, v = (a[rank * per_rank:(rank + 1) * per_rank] for a in inputs())
    qd, kd, vd = (runtime.upload(a) for a in (q, k, v))
    whole = runtime.empty(BH * T * D * 2)
    lse = runtime.empty(per_rank * T * 4)
    mine = whole.ptr + rank * per_rank * T * D * 2  # the shard is computed straight into its slice of the gathered tensor
    check(L.limn_b200_sdpa_fwd(qd.ptr, kd.ptr, vd.ptr, None, mine, lse.ptr, 2, per_rank, T, T, D, D, 1, D**-0.5, None), "sdpa")
    check(L.limn_b200_nccl_all_gather(mine, whole.ptr, per_rank * T * D * 2, None), "gathering the shards")
    runtime.synchronize()
    assert runtime.device_status() == 0
    np.save(scratch / f"whole_{rank}.npy", runtime.download(whole, np.uint16, (BH, T, D)))
    check(L.limn_b200_nccl_destroy(), "leaving the communicator")


if __name__ == "__main__":
    rank_main(int(sys.argv[1]), int(sys.argv[2]), Path(sys.argv[3]))
else:
    import pytest
    from conftest import parity

    from oracle import sdpa_oracle as oracle

    @pytest.mark.gpu
    def test_two_ranks_gather_their_shards_over_nccl(tmp_path):
        from limn_b200 import runtime

        if runtime.device_count() < 2:
            pytest.skip("needs two GPUs")
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        ranks = [subprocess.Popen([sys.executable, __file__, str(r), "2", str(tmp_path)], env=env, stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True) for r in range(2)]
        outputs = []
        for proc in ranks:
            try:
                outputs.append(proc.communicate(timeout=300)[0])
            except subprocess.TimeoutExpired:
                proc.kill()  # the exact process started above
                outputs.append(proc.communicate()[0])
        assert all(proc.returncode == 0 for proc in ranks), "\n".join(o[-1500:] for o in outputs)
        q, k, v = inputs()
        want, _ = oracle.sdpa_forward(q, k, v, causal=True, scale=D**-0.5)
        gathered = [np.load(tmp_path / f"whole_{r}.npy").view(BF16) for r in range(2)]
        np.testing.assert_array_equal(gathered[0].view(np.uint16), gathered[1].view(np.uint16))  # every rank holds the same tensor
        parity(gathered[0], want, 2e-2, "gathered O over 2 ranks")
