"""Benchmark of the fused-attention path on B200: TFLOP/s of `sdpa` (and, for the workloads
that have a backward, `sdpa` + `sdpa_bwd_q` + `sdpa_bwd_kv`) through the C ABI.

    python bench.py                                  # 1 GPU, default workload, a few minutes
    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 3
    python bench.py --impl reference                 # the CPU restatement of limn's numpy kernels

One step is one pass of the hot path over the whole workload: every (batch, head) problem of
the named configuration, forward only or forward plus both backward kernels. The (batch,
head) problems are independent, so at N GPUs rank r takes problems [r*BH/N, (r+1)*BH/N) and
no collective sits on the data path; NCCL is used once, after the timed region, to gather
the output shards. Rank 0 prints one JSON line.

Inputs are synthetic and seeded per problem (so a shard holds the same values whatever N
is): Q, K, V, dO drawn in float32 and rounded to bfloat16, with the scales each workload
states. torch is used here for device memory and torch.distributed only; the kernels are
reached through limn_b200's ctypes binding and timed with CUDA events on the stream they
are launched on (the legacy default stream, which is also torch's).
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import ml_dtypes
import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
BF16 = np.dtype(ml_dtypes.bfloat16)

# name -> (B, H, S, D, causal, backward?, q/k multiplier, v kind, seed, description)
WORKLOADS = {
    "gpt_layer": (32, 8, 256, 64, True, True, 1.0, "normal", 2, "byte-level GPT attention layer B=32 H=8 S=256 D=64 causal bf16, fwd+bwd"),
    "prefill_4k": (8, 32, 4096, 128, True, False, 0.5, "half", 3, "long-context causal prefill B=8 H=32 S=4096 D=128 bf16, forward only"),
    "encoder_2k": (16, 16, 2048, 64, False, True, 1.0, "normal", 4, "non-causal encoder B=16 H=16 S=2048 D=64 bf16, fwd+bwd"),
    "ragged_3000": (4, 40, 3000, 128, True, True, 2.0, "uniform", 5, "ragged tail B=4 H=40 S=3000 D=128 causal bf16 sharp softmax, fwd+bwd"),
}
DEFAULT_WORKLOAD = "prefill_4k"
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}


def fwd_flops(bh: int, s: int, d: int, causal: bool) -> float:
    """4 * BH * S^2 * D, halved for causal by convention: the two GEMMs of the forward."""
    return 4.0 * bh * s * s * d * (0.5 if causal else 1.0)


def problem_inputs(workload: str, problem: int):
    """Q, K, V, dO of one (batch, head) problem as (S, D) bfloat16 arrays, seeded by (workload seed, problem)."""
    _, _, s, d, _, _, mul, v_kind, seed, _ = WORKLOADS[workload]
    rng = np.random.default_rng([seed, problem])
    q = (rng.standard_normal((s, d), dtype=np.float32) * mul).astype(BF16)
    k = (rng.standard_normal((s, d), dtype=np.float32) * mul).astype(BF16)
    if v_kind == "uniform":
        v = rng.uniform(-1.0, 1.0, (s, d)).astype(np.float32).astype(BF16)
    else:
        v = (rng.standard_normal((s, d), dtype=np.float32) * (0.5 if v_kind == "half" else 1.0)).astype(BF16)
    do = rng.standard_normal((s, d), dtype=np.float32).astype(BF16)
    return q, k, v, do


def shard_inputs(workload: str, first: int, count: int, want_do: bool):
    s, d = WORKLOADS[workload][2], WORKLOADS[workload][3]
    arrays = [np.empty((count, s, d), dtype=BF16) for _ in range(4 if want_do else 3)]
    for i in range(count):
        for dst, src in zip(arrays, problem_inputs(workload, first + i)):
            dst[i] = src
    return arrays


def shard_range(bh: int, rank: int, world: int) -> tuple[int, int]:
    """(first problem, count) of rank's contiguous share of bh independent (batch, head) problems."""
    if bh % world:
        raise ValueError(f"{bh} (batch, head) problems do not split evenly over {world} ranks")
    per_rank = bh // world
    return rank * per_rank, per_rank


def reduce_max(value: float, dist, device) -> float:
    """The slowest rank's time: every multi-GPU number is the max over ranks."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    import torch

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def forward_traffic(workload: str, problems: int):
    """DRAM bytes (read + write) of one forward launch, from the ncu captures summarised under profiles/:
    measured on a subset of the workload's problems and scaled by the problem count, to which it is
    proportional (every problem's tensors cross HBM once). None where no capture exists."""
    per_problem = {"prefill_4k": (202.346496e6 + 47.651328e6) / 64, "encoder_2k": (102.376448e6 + 18.868224e6) / 128}
    return per_problem[workload] * problems if workload in per_problem else None


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 50 ms while running."""

    FIELDS = "timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.marks: list[float] = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def mark(self) -> None:
        """Start (first call) or end (second call) of the region whose samples count."""
        self.marks.append(time.time())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()  # the exact process started above
        self.proc.wait()
        self.file.flush()
        from datetime import datetime

        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.count(",") >= 6]
        os.unlink(self.file.name)
        lo, hi = (self.marks + [0.0, 1e18])[:2] if len(self.marks) >= 2 else (0.0, 1e18)
        clocks, reasons, top = [], set(), None
        for row in rows:
            try:
                stamp = datetime.strptime(row[0].strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if not (lo - 0.1 <= stamp <= hi + 0.1):
                    continue
                clocks.append(float(row[1]))
                top = float(row[2])
            except ValueError:
                continue
            for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), row[3:7]):
                if flag.strip().lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(clocks)) if clocks else None, "sm_max_mhz": top, "reasons": sorted(reasons), "samples": len(clocks)}


# ---------------------------------------------------------------- the CPU arm


def cpu_pass(workload: str, problems: list[int]) -> tuple[float, float]:
    """Run the CPU oracle over the given problems (forward, plus both backward ops where the
    workload has them); returns (seconds, flops credited)."""
    from oracle import sdpa_oracle as oracle

    _, _, s, d, causal, backward, *_ = WORKLOADS[workload]
    scale = d ** -0.5
    start = time.perf_counter()
    for problem in problems:
        q, k, v, do = problem_inputs(workload, problem)
        out, lse = oracle.sdpa_forward(q, k, v, causal=causal, scale=scale)
        if backward:
            delta = oracle.row_delta(do, out)
            oracle.sdpa_backward_q(q, k, v, do, lse, delta, causal=causal, scale=scale)
            oracle.sdpa_backward_kv(q, k, v, do, lse, delta, causal=causal, scale=scale)
    seconds = time.perf_counter() - start
    return seconds, fwd_flops(len(problems), s, d, causal) * (3.5 if backward else 1.0)


def cpu_sample_size(workload: str, target_seconds: float) -> int:
    """How many (b, h) problems make about target_seconds of CPU work, from one timed problem."""
    seconds, _ = cpu_pass(workload, [0])
    bh = WORKLOADS[workload][0] * WORKLOADS[workload][1]
    return max(1, min(bh, int(target_seconds / max(seconds, 1e-4))))


def reference_arm(args) -> None:
    """The reference's CPU implementation of the path, restated in oracle/ (limn/sdpa.py is
    Python over numpy/BLAS and is not on the GPU box), on a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    workload = args.workload
    b, h, s, d, causal, backward, *_ = WORKLOADS[workload]
    sample = cpu_sample_size(workload, min(6.0, 90.0 / max(args.steps, 1)))
    problems = list(range(sample))
    for _ in range(min(args.warmup, 1)):
        cpu_pass(workload, problems[:1])
    total_seconds, total_flops = 0.0, 0.0
    for _ in range(args.steps):
        seconds, flops = cpu_pass(workload, problems)
        total_seconds += seconds
        total_flops += flops
    value = total_flops / total_seconds / 1e12
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": "sdpa TFLOP/s (forward, or forward+backward where the workload has one)",
        "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": min(args.warmup, 1),
        "ms_per_step": total_seconds / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16 storage, f32 arithmetic", "data": "synthetic",
        "config": {"workload": workload, "describes": WORKLOADS[workload][-1], "pass": "fwd+bwd" if backward else "fwd"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{sample} of {b * h} (batch, head) problems per step, numpy/BLAS threads = host cores"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------- the GPU arm


class Shard:
    """One rank's problems of a workload, resident on its GPU as torch tensors."""

    def __init__(self, workload: str, first: int, count: int, torch, device, force_backward: bool = False):
        from limn_b200._lib import lib

        self.lib = lib()
        self.workload = workload
        b, h, s, d, causal, backward, *_ = WORKLOADS[workload]
        backward = backward or force_backward
        self.count, self.s, self.d, self.causal, self.backward = count, s, d, causal, backward
        self.scale = d ** -0.5
        host = shard_inputs(workload, first, count, backward)
        self.pinned = [torch.from_numpy(a.view(np.int16)).pin_memory() for a in host]
        self.dev = [t.to(device, non_blocking=False) for t in self.pinned]
        shape = (count, s, d)
        self.out = torch.empty(shape, dtype=torch.int16, device=device)
        self.lse = torch.empty((count, s), dtype=torch.float32, device=device)
        self.out_host = torch.empty(shape, dtype=torch.int16).pin_memory()
        self.lse_host = torch.empty((count, s), dtype=torch.float32).pin_memory()
        if backward:
            self.delta = torch.empty((count, s), dtype=torch.float32, device=device)
            self.dq, self.dk, self.dv = (torch.empty(shape, dtype=torch.int16, device=device) for _ in range(3))
            self.grad_host = [torch.empty(shape, dtype=torch.int16).pin_memory() for _ in range(3)]
        self.launches = 0
        self.pipeline = None
        # "bthd": the same bytes read as one batch of `count` heads held token-major, (1, s, count, d), through
        # the layout entry points (the values are random, so any reading of them is as good a workload)
        self.layout = "bhtd"

    def _check(self, code: int, doing: str) -> None:
        if code != 0:
            raise RuntimeError(f"limn_b200: {doing}: {self.lib.limn_b200_last_error().decode()}")
        self.launches += self.lib.limn_b200_last_launch_count()

    def forward(self) -> None:
        q, k, v = (t.data_ptr() for t in self.dev[:3])
        if self.layout == "bthd":
            self._check(self.lib.limn_b200_sdpa_fwd_layout(q, k, v, None, self.out.data_ptr(), self.lse.data_ptr(), 1, 2, 1, self.count,
                                                           self.s, self.s, self.d, self.d, int(self.causal), self.scale, None), "sdpa")
            return
        self._check(self.lib.limn_b200_sdpa_fwd(q, k, v, None, self.out.data_ptr(), self.lse.data_ptr(), 2, self.count, self.s,
                                                self.s, self.d, self.d, int(self.causal), self.scale, None), "sdpa")

    def backward_pass(self) -> None:
        q, k, v, do = (t.data_ptr() for t in self.dev[:4])
        if self.layout == "bthd":
            tail = (1, 2, 1, self.count, self.s, self.s, self.d, self.d, int(self.causal), self.scale, None)
            self._check(self.lib.limn_b200_sdpa_delta_layout(self.out.data_ptr(), do, self.delta.data_ptr(), 1, 2, 1, self.count, self.s, self.d, None), "row dot")
            self._check(self.lib.limn_b200_sdpa_bwd_q_layout(q, k, v, do, self.lse.data_ptr(), self.delta.data_ptr(), None, self.dq.data_ptr(), *tail), "sdpa_bwd_q")
            self._check(self.lib.limn_b200_sdpa_bwd_kv_layout(q, k, v, do, self.lse.data_ptr(), self.delta.data_ptr(), None, self.dk.data_ptr(),
                                                              self.dv.data_ptr(), *tail), "sdpa_bwd_kv")
            return
        tail = (2, self.count, self.s, self.s, self.d, self.d, int(self.causal), self.scale, None)
        self._check(self.lib.limn_b200_sdpa_delta(self.out.data_ptr(), do, self.delta.data_ptr(), 2, self.count * self.s, self.d, None), "row dot")
        self._check(self.lib.limn_b200_sdpa_bwd_q(q, k, v, do, self.lse.data_ptr(), self.delta.data_ptr(), None, self.dq.data_ptr(), *tail), "sdpa_bwd_q")
        self._check(self.lib.limn_b200_sdpa_bwd_kv(q, k, v, do, self.lse.data_ptr(), self.delta.data_ptr(), None, self.dk.data_ptr(),
                                                   self.dv.data_ptr(), *tail), "sdpa_bwd_kv")

    def step(self) -> None:
        self.forward()
        if self.backward:
            self.backward_pass()

    def step_from_host(self) -> tuple[int, int]:
        """One step with host buffers, through limn_b200.hostio.HostPipeline: inputs come up from pinned
        memory and results go back down to pinned memory, chunk by chunk, the copies overlapped with the
        kernels on three streams. Returns (bytes uploaded, bytes downloaded)."""
        if self.pipeline is None:
            from limn_b200.hostio import HostPipeline

            self.pipeline = HostPipeline(self.count, self.s, self.d, causal=self.causal, backward=self.backward, chunk=16)
            self.host_in = [t.numpy() for t in self.pinned]
            self.host_out = [self.out_host.numpy()] + ([t.numpy() for t in self.grad_host] if self.backward else [])
            self.host_lse = self.lse_host.numpy()
        q, k, v = self.host_in[:3]
        extra = dict(do=self.host_in[3], dq=self.host_out[1], dk=self.host_out[2], dv=self.host_out[3]) if self.backward else {}
        up, down = self.pipeline(q, k, v, self.host_out[0], self.host_lse, **extra)
        self.launches += self.pipeline.launches
        return up, down

    def flops_per_step(self) -> float:
        return fwd_flops(self.count, self.s, self.d, self.causal) * (3.5 if self.backward else 1.0)


def timed(shard: Shard, steps: int, body) -> float:
    """Milliseconds for `steps` calls of body(), by CUDA events on the launch stream."""
    from limn_b200 import runtime

    start, stop = runtime.Event(), runtime.Event()
    start.record()
    for _ in range(steps):
        body()
    stop.record()
    runtime.synchronize()
    return stop.ms_since(start)


def other_workloads(args, main: str, world: int, rank: int, torch, device, barrier, max_over_ranks) -> dict:
    """The remaining BASELINE configurations, device-resident, forward and (where the workload has one)
    forward+backward, each timed the same way as the main workload but with fewer steps. They ride along
    as context for the headline number; the parity of every one of them is the tests' business."""
    found = {}
    peak, _ = peaks()
    tensor_peak = float(peak.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    for name, (b, h, s, d, causal, backward, *_rest) in WORKLOADS.items():
        if name == main or (b * h) % world:
            continue
        first, count = shard_range(b * h, rank, world)
        shard = Shard(name, first, count, torch, device)
        steps = max(3, min(args.steps, 10))
        for _ in range(3):
            shard.step()
        barrier()
        fwd_ms = max_over_ranks(timed(shard, steps, shard.forward)) / steps
        entry = {"fwd_ms": fwd_ms, "fwd_tflops": fwd_flops(b * h, s, d, causal) / (fwd_ms * 1e-3) / 1e12}
        entry["fwd_pct_of_measured_peak"] = 100 * entry["fwd_tflops"] / world / tensor_peak
        if backward:
            barrier()
            step_ms = max_over_ranks(timed(shard, steps, shard.step)) / steps
            entry["fwd_bwd_ms"] = step_ms
            entry["fwd_bwd_tflops"] = 3.5 * fwd_flops(b * h, s, d, causal) / (step_ms * 1e-3) / 1e12
            entry["fwd_bwd_pct_of_measured_peak"] = 100 * entry["fwd_bwd_tflops"] / world / tensor_peak
            entry["includes"] = "sdpa + row dot (delta) + sdpa_bwd_q + sdpa_bwd_kv; credited 3.5x forward flops, executed 4.5x"
        # the same step with the operands held token-major, (batch, t, heads, hd), through the layout entry points,
        # and what the permute copies that layout makes unnecessary cost (torch, one per operand and result)
        shard.layout = "bthd"
        for _ in range(3):
            shard.step()
        barrier()
        entry["token_major_ms"] = max_over_ranks(timed(shard, steps, shard.step)) / steps
        shard.layout = "bhtd"
        tensors = shard.dev[:4 if backward else 3] + [shard.out] + ([shard.dq, shard.dk, shard.dv] if backward else [])

        def permute_copies():
            for t in tensors:
                t.view(1, s, count, d).transpose(1, 2).contiguous()

        permute_copies()
        barrier()
        entry["permute_copies_ms"] = max_over_ranks(timed(shard, steps, permute_copies)) / steps
        found[name] = entry
        del shard
        torch.cuda.empty_cache()
    return found


def gpu_arm(args) -> None:
    import torch
    import torch.distributed as dist

    from limn_b200 import runtime

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    runtime.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout: rank 0 prints exactly one line
        dist.init_process_group("nccl", device_id=device)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        return reduce_max(x, dist if world > 1 else None, device)

    workload = args.workload
    b, h, s, d, causal, backward, *_ = WORKLOADS[workload]
    bh = b * h
    try:
        first_problem, per_rank = shard_range(bh, rank, world)
    except ValueError as err:
        raise SystemExit(str(err))
    sampler = ClockSampler(local) if rank == 0 else None  # started early: nvidia-smi takes a second or two to produce its first row
    shard = Shard(workload, first_problem, per_rank, torch, device)
    peak, peak_kind = peaks()

    # ---- device-resident throughput ----
    for _ in range(max(args.warmup, 3)):
        shard.step()
    barrier()
    shard.launches = 0
    if sampler:
        sampler.mark()
    ms = timed(shard, args.steps, shard.step)
    barrier()
    launches = shard.launches
    ms = max_over_ranks(ms)
    total_flops = fwd_flops(bh, s, d, causal) * (3.5 if backward else 1.0)
    value = total_flops * args.steps / (ms * 1e-3) / 1e12

    # dominant kernel alone (the forward), for the roofline entry
    barrier()
    fwd_ms = max_over_ranks(timed(shard, args.steps, shard.forward)) / args.steps
    fwd_rate = fwd_flops(per_rank, s, d, causal) / (fwd_ms * 1e-3) / 1e12

    # ---- end to end with host buffers ----
    e2e_steps = max(2, min(args.steps, 5))
    shard.step_from_host()
    barrier()
    up = down = 0

    def from_host() -> None:
        nonlocal up, down
        up, down = shard.step_from_host()

    e2e_ms = max_over_ranks(timed(shard, e2e_steps, from_host))
    e2e_value = total_flops * e2e_steps / (e2e_ms * 1e-3) / 1e12
    if sampler:
        sampler.mark()
    clocks = sampler.stop() if sampler else None  # samples taken between the first timed launch and the last

    # ---- the one collective: gather the output shards (outside the timed region) ----
    gather_ms = None
    if world > 1:
        whole = torch.empty((bh, s, d), dtype=torch.int16, device=device)
        barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        dist.all_gather_into_tensor(whole.view(torch.bfloat16), shard.out.view(torch.bfloat16))
        t1.record()
        torch.cuda.synchronize()
        gather_ms = max_over_ranks(t0.elapsed_time(t1))

    others = other_workloads(args, workload, world, rank, torch, device, barrier, max_over_ranks) if args.others else None

    status = runtime.device_status()
    if status:
        raise SystemExit(f"a kernel gave up on a bounded wait (status 0x{status:08x}); no number is reported")

    if rank == 0:
        # spot parity: problem 0 of this shard against the CPU oracle
        from oracle import sdpa_oracle as oracle

        q, k, v, do = problem_inputs(workload, 0)
        want_out, want_lse = oracle.sdpa_forward(q, k, v, causal=causal, scale=d ** -0.5)
        got_out = shard.out[0].cpu().numpy().view(BF16).astype(np.float32)
        got_lse = shard.lse[0].cpu().numpy()
        parity = {"problem": 0, "max_abs_out": float(np.abs(got_out - want_out.astype(np.float32)).max()),
                  "max_abs_lse": float(np.abs(got_lse - want_lse[..., 0]).max())}

        sample = cpu_sample_size(workload, 12.0)
        cpu_seconds, cpu_flops = cpu_pass(workload, list(range(sample)))
        tensor_peak = float(peak.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        line = {
            "metric": "sdpa TFLOP/s (forward, or forward+backward where the workload has one)",
            "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 operands, f32 accumulate", "data": "synthetic",
            "config": {"workload": workload, "describes": WORKLOADS[workload][-1], "pass": "fwd+bwd" if backward else "fwd",
                       "problems_per_rank": per_rank, "sharding": "(batch, head) problems split evenly over ranks, no data-path collective",
                       "l2": "inputs larger than L2" if per_rank * s * d * 2 * 3 > 126e6 else "inputs smaller than L2 (resident between steps)"},
            "pct_of_peak": {"of_measured_burst": 100 * value / world / tensor_peak,
                            "of_measured_sustained": 100 * value / world / float(peak.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"])),
                            "of_nominal_2250": 100 * value / world / 2250.0},
            "roofline": {"bound": "tensor", "kernel": "sdpa_fwd_kernel", "achieved": fwd_rate, "peak": tensor_peak, "unit": "TFLOP/s",
                         "frac": fwd_rate / tensor_peak, "peak_kind": f"{peak_kind} burst (kernel timed alone, {args.steps} launches)",
                         "traffic": forward_traffic(workload, per_rank), "ms_per_launch": fwd_ms},
            "cpu_baseline": {"value": cpu_flops / cpu_seconds / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count() or 1, "kind": "port",
                             "sample": f"{sample} of {bh} (batch, head) problems, {cpu_seconds:.1f} s"},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": up * world, "d2h_bytes_per_step": down * world,
                    "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": launches * world,
            "clocks": clocks,
            "gather_ms": gather_ms,
            "parity": parity,
            "others": others,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def profile_case(args) -> None:
    """For profiler captures: the first N problems of a workload, each kernel of the path launched
    `--steps` times after one warm-up pass, nothing timed and nothing printed but a status line.
    `ncu -k regex:sdpa_ ...  python bench.py --profile N --workload W [--backward]` then sees a small,
    bounded case of the same kernels on the same seeded inputs."""
    import torch

    from limn_b200 import runtime

    torch.cuda.set_device(0)
    runtime.set_device(0)
    b, h, s, d, causal, backward, *_ = WORKLOADS[args.workload]
    count = min(args.profile, b * h)
    shard = Shard(args.workload, 0, count, torch, torch.device("cuda", 0), force_backward=args.backward)
    shard.step()
    for _ in range(args.steps):
        shard.step()
    torch.cuda.synchronize()
    print(json.dumps({"profiled": args.workload, "problems": count, "backward": shard.backward, "device_status": runtime.device_status()}))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("limn_b200", "reference"), default="limn_b200")
    parser.add_argument("--workload", choices=sorted(WORKLOADS), default=DEFAULT_WORKLOAD)
    parser.add_argument("--profile", type=int, default=0, metavar="N", help="launch the kernels over the first N problems and exit (for ncu)")
    parser.add_argument("--backward", action="store_true", help="with --profile: run the backward kernels even for a forward-only workload")
    parser.add_argument("--no-others", dest="others", action="store_false", help="time only the named workload")
    args = parser.parse_args()
    if args.profile:
        profile_case(args)
    elif args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
