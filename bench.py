"""Benchmark of the fused-attention path on B200: TFLOP/s of `sdpa` (and, for the workloads
that have a backward, `sdpa` + `sdpa_bwd_q` + `sdpa_bwd_kv`) through the C ABI.

    python bench.py                                  # 1 GPU, default workload, a few minutes
    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 3
    python bench.py --impl reference                 # limn's own numpy kernels on the host cores (its CPU path)
    python bench.py --limn-arm prefill_4k            # limn itself on the GPU: its NVRTC kernels, then ours installed

One step is one pass of the hot path over the whole workload: every (batch, head) problem of
the named configuration, forward only or forward plus both backward kernels. The (batch,
head) problems are independent, so at N GPUs rank r takes problems [r*BH/N, (r+1)*BH/N) and
no collective sits on the data path; NCCL gathers the output shards, either after the timed
region or, for the "gathered" figure, chunk by chunk on a side stream while later chunks
compute. Rank 0 prints one JSON line, the last line of its standard output.

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
METRIC = "sdpa TFLOP/s (forward, or forward+backward where the workload has one)"
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


def forward_traffic(workload: str, problems: int) -> tuple[float | None, str]:
    """DRAM bytes (read + write) of one forward launch, from the ncu captures summarised under profiles/:
    measured on a subset of the workload's problems and scaled by the problem count, to which it is
    proportional (every problem's tensors cross HBM once). (None, why) where no capture exists."""
    captured = {
        # workload: (problems in the capture, dram bytes read, dram bytes written, what the capture was)
        "prefill_4k": (128, 406.098944e6, 121.099264e6,
                       "128-problem capture (402.7 MB of Q, K, V; 136.3 MB of O and L, more than L2 holds): reads are the inputs "
                       "once; 15 MB of the output had not left L2 when the counters stopped, so the write side is a lower bound"),
        "encoder_2k": (128, 102.376448e6, 18.868224e6, "128-problem capture; its 34 MB of output fit in L2, so the write side is a lower bound"),
    }
    if workload not in captured:
        return None, "no ncu capture of this workload"
    n, read, written, note = captured[workload]
    return (read + written) / n * problems, note


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 50 ms while running; regions of
    interest are bracketed with begin(name) / end(name) and summarised separately."""

    FIELDS = "timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw"

    def __init__(self, index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.regions: dict[str, list[float]] = {}
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def begin(self, name: str) -> None:
        self.regions[name] = [time.time()]

    def end(self, name: str) -> None:
        self.regions[name].append(time.time())

    def stop(self) -> dict:
        """{region: {"sm_mhz": median under load, "sm_max_mhz", "reasons", "samples"}}"""
        if self.proc is None:
            return {name: {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]} for name in self.regions}
        time.sleep(0.25)
        self.proc.terminate()  # the exact process started above
        self.proc.wait()
        self.file.flush()
        from datetime import datetime

        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.count(",") >= 6]
        os.unlink(self.file.name)
        found = {}
        for name, marks in self.regions.items():
            lo, hi = marks[0], (marks[1] if len(marks) > 1 else 1e18)
            clocks, power, reasons, top = [], [], set(), None
            for row in rows:
                try:
                    stamp = datetime.strptime(row[0].strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    if not (lo - 0.1 <= stamp <= hi + 0.1):
                        continue
                    clocks.append(float(row[1]))
                    top = float(row[2])
                    if len(row) > 7:
                        power.append(float(row[7]))
                except ValueError:
                    continue
                for reason, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), row[3:7]):
                    if flag.strip().lower().startswith("active"):
                        reasons.add(reason)
            found[name] = {"sm_mhz": float(np.median(clocks)) if clocks else None, "sm_max_mhz": top, "reasons": sorted(reasons),
                           "samples": len(clocks), "power_w_max": max(power) if power else None}
        return found


# ---------------------------------------------------------------- the CPU arm


STAGED_LIMN = ROOT / "baseline" / "_ref"


def limn_on_path() -> bool:
    """Put the staged copy of limn (baseline/_ref, made by __graft_entry__.build() where the reference is at hand)
    on sys.path; False when there is none."""
    if not (STAGED_LIMN / "limn" / "sdpa.py").is_file():
        return False
    if str(STAGED_LIMN) not in sys.path:
        sys.path.insert(0, str(STAGED_LIMN))
    return True


def cpu_kernels():
    """The CPU implementation of the path and what it is: limn's own numpy kernels (limn/sdpa.py:91-203, the
    functions its numpy device dispatches the three CUSTOM ops to) when limn is staged here, "reference"; else
    the restatement under oracle/, "port". Returns (forward, backward_q, backward_kv, kind)."""
    if limn_on_path():
        from limn import sdpa as ref

        return ref.sdpa, ref.sdpa_backward_q, ref.sdpa_backward_kv, "reference"
    from oracle import sdpa_oracle as oracle

    return oracle.sdpa_forward, oracle.sdpa_backward_q, oracle.sdpa_backward_kv, "port"


def cpu_pass(workload: str, problems: list[int]) -> tuple[float, float]:
    """Run the CPU implementation over the given problems (forward, plus both backward ops where the
    workload has them); returns (seconds, flops credited)."""
    forward, backward_q, backward_kv, _ = cpu_kernels()
    _, _, s, d, causal, backward, *_ = WORKLOADS[workload]
    scale = d ** -0.5
    start = time.perf_counter()
    for problem in problems:
        q, k, v, do = problem_inputs(workload, problem)
        out, lse = forward(q, k, v, causal=causal, scale=scale)
        if backward:
            delta = (do.astype(np.float32) * out.astype(np.float32)).sum(axis=-1, keepdims=True)  # limn/tensor.py:705-706
            backward_q(q, k, v, do, lse, delta, causal=causal, scale=scale)
            backward_kv(q, k, v, do, lse, delta, causal=causal, scale=scale)
    seconds = time.perf_counter() - start
    return seconds, fwd_flops(len(problems), s, d, causal) * (3.5 if backward else 1.0)


def cpu_sample_size(workload: str, target_seconds: float) -> int:
    """How many (b, h) problems make about target_seconds of CPU work, from one timed problem."""
    seconds, _ = cpu_pass(workload, [0])
    bh = WORKLOADS[workload][0] * WORKLOADS[workload][1]
    return max(1, min(bh, int(target_seconds / max(seconds, 1e-4))))


def c_device_pass(workload: str) -> dict | None:
    """limn's C backend on one (batch, head) problem of the workload: it registers no CUSTOM kernel
    (limn/backend_c.py:242-264), so Tensor.attention runs there in its composed form (limn/tensor.py:673-676),
    lowered to single-threaded C, float32 only, with the t x t scores materialised. One problem bounds both the
    time and the memory; the first call (which compiles) is not timed. None without limn or a C compiler."""
    if not limn_on_path():
        return None
    try:
        import limn
        from limn import backend_c

        if not backend_c.has_cc():
            return None
        _, _, s, d, causal, backward, *_ = WORKLOADS[workload]
        q, k, v, do = (a.astype(np.float32) for a in problem_inputs(workload, 0))
        limn.set_device("c")
        try:
            def once() -> float:
                tq, tk, tv = (limn.Tensor(a, requires_grad=backward) for a in (q, k, v))
                start = time.perf_counter()
                out = tq.attention(tk, tv, causal=causal)
                if backward:
                    limn.realize(*limn.grad((out * limn.Tensor(do)).sum(), [tq, tk, tv]))
                else:
                    out.realize()
                return time.perf_counter() - start

            once()
            seconds = once()
        finally:
            limn.set_device("numpy")
        flops = fwd_flops(1, s, d, causal) * (3.5 if backward else 1.0)
        return {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": 1, "seconds": seconds,
                "sample": "1 (batch, head) problem, float32 copies of the same values, composed attention (no CUSTOM kernel on this device)"}
    except Exception as err:  # a baseline that cannot run is reported, not fatal
        return {"unavailable": f"{type(err).__name__}: {err}"[:200]}


def reference_arm(args) -> None:
    """The reference's CPU implementation of the path on the host cores: limn's own numpy kernels
    (BLAS-threaded) from the staged copy of limn, on a bounded sample of the workload per step; beside it, once,
    its C backend on one problem. Without a staged limn the restatement under oracle/ stands in (kind "port")."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    workload = args.workload
    b, h, s, d, causal, backward, *_ = WORKLOADS[workload]
    kind = cpu_kernels()[3]
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
        "impl": "reference", "metric": METRIC,
        "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": min(args.warmup, 1),
        "ms_per_step": total_seconds / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16 storage, f32 arithmetic", "data": "synthetic",
        "config": {"workload": workload, "describes": WORKLOADS[workload][-1], "pass": "fwd+bwd" if backward else "fwd"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": kind,
                         "sample": f"{sample} of {b * h} (batch, head) problems per step, limn.sdpa on numpy/BLAS, threads = host cores"},
        "c_device": c_device_pass(workload),
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
        # True: the row dot as a kernel of its own before the dQ pass (what limn's frontend schedules today); False: inside it
        self.separate_delta = False

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

    def forward_range(self, first: int, count: int) -> None:
        """The forward over problems [first, first + count) of the shard as a launch of its own."""
        step = self.s * self.d * 2
        q, k, v = (t.data_ptr() + first * step for t in self.dev[:3])
        self._check(self.lib.limn_b200_sdpa_fwd(q, k, v, None, self.out.data_ptr() + first * step, self.lse.data_ptr() + first * self.s * 4,
                                                2, count, self.s, self.s, self.d, self.d, int(self.causal), self.scale, None), "sdpa")

    def backward_pass(self) -> None:
        q, k, v, do = (t.data_ptr() for t in self.dev[:4])
        if self.layout == "bthd":
            tail = (1, 2, 1, self.count, self.s, self.s, self.d, self.d, int(self.causal), self.scale, None)
            self._check(self.lib.limn_b200_sdpa_bwd_q_fused_layout(q, k, v, self.out.data_ptr(), do, self.lse.data_ptr(), None, self.dq.data_ptr(),
                                                                   self.delta.data_ptr(), *tail), "sdpa_bwd_q")
            self._check(self.lib.limn_b200_sdpa_bwd_kv_layout(q, k, v, do, self.lse.data_ptr(), self.delta.data_ptr(), None, self.dk.data_ptr(),
                                                              self.dv.data_ptr(), *tail), "sdpa_bwd_kv")
            return
        tail = (2, self.count, self.s, self.s, self.d, self.d, int(self.causal), self.scale, None)
        if self.separate_delta:
            self._check(self.lib.limn_b200_sdpa_delta(self.out.data_ptr(), do, self.delta.data_ptr(), 2, self.count * self.s, self.d, None), "row dot")
            self._check(self.lib.limn_b200_sdpa_bwd_q(q, k, v, do, self.lse.data_ptr(), self.delta.data_ptr(), None, self.dq.data_ptr(), *tail), "sdpa_bwd_q")
        else:
            self._check(self.lib.limn_b200_sdpa_bwd_q_fused(q, k, v, self.out.data_ptr(), do, self.lse.data_ptr(), None, self.dq.data_ptr(),
                                                            self.delta.data_ptr(), *tail), "sdpa_bwd_q")
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

            self.pipeline = HostPipeline(self.count, self.s, self.d, causal=self.causal, backward=self.backward)
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


# Algorithmic HBM bytes of each kernel of the path per (batch, head) problem of S tokens and head dim D in 16-bit
# storage (every operand and result crosses HBM once; L and delta are float32 per row):
#   sdpa        reads Q, K, V, writes O, L                    8 S D + 4 S
#   delta       reads O, dO, writes delta                     4 S D + 4 S   (inside sdpa_bwd_q when fused; the bytes are the same)
#   sdpa_bwd_q  reads Q, K, V, dO, L, delta, writes dQ       10 S D + 8 S
#   sdpa_bwd_kv reads Q, K, V, dO, L, delta, writes dK, dV   12 S D + 8 S
def hbm_bytes(kernel: str, bh: int, s: int, d: int) -> float:
    per = {"sdpa": 8 * s * d + 4 * s, "delta": 4 * s * d + 4 * s, "sdpa_bwd_q": 10 * s * d + 8 * s, "sdpa_bwd_kv": 12 * s * d + 8 * s}
    return float(per[kernel]) * bh


def other_workloads(args, main: str, world: int, rank: int, torch, device, barrier, max_over_ranks) -> dict:
    """The remaining BASELINE configurations, device-resident, forward and (where the workload has one)
    forward+backward, each timed the same way as the main workload (best of three trials) but with fewer
    steps. They ride along as context for the headline number; the parity of every one of them is the tests'
    business."""
    found = {}
    peak, _ = peaks()
    tensor_peak = float(peak.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    hbm_peak = float(peak.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    for name, (b, h, s, d, causal, backward, *_rest) in WORKLOADS.items():
        if name == main or (b * h) % world:
            continue
        first, count = shard_range(b * h, rank, world)
        shard = Shard(name, first, count, torch, device)
        steps = max(3, min(args.steps, 10))
        for _ in range(3):
            shard.step()

        def best(body) -> float:
            trials = []
            for _ in range(3):
                barrier()
                time.sleep(args.rest_seconds)
                barrier()
                trials.append(max_over_ranks(timed(shard, steps, body)) / steps)
            return min(trials)

        fwd_ms = best(shard.forward)
        entry = {"fwd_ms": fwd_ms, "fwd_tflops": fwd_flops(b * h, s, d, causal) / (fwd_ms * 1e-3) / 1e12}
        entry["fwd_pct_of_measured_peak"] = 100 * entry["fwd_tflops"] / world / tensor_peak
        if backward:
            step_ms = best(shard.step)
            entry["fwd_bwd_ms"] = step_ms
            entry["fwd_bwd_tflops"] = 3.5 * fwd_flops(b * h, s, d, causal) / (step_ms * 1e-3) / 1e12
            entry["fwd_bwd_pct_of_measured_peak"] = 100 * entry["fwd_bwd_tflops"] / world / tensor_peak
            entry["includes"] = "sdpa + sdpa_bwd_q with the row dot (delta) computed inside it + sdpa_bwd_kv; credited 3.5x forward flops, executed 4.5x"
            shard.separate_delta = True
            entry["fwd_bwd_ms_with_a_separate_row_dot_kernel"] = best(shard.step)
            shard.separate_delta = False
        if s * 2 < 1024:
            # a short-sequence workload is bound by HBM and launch latency, not by the tensor pipe: the same
            # times against the bytes each kernel has to move (hbm_bytes above) and the measured copy bandwidth
            moved = hbm_bytes("sdpa", count, s, d)
            entry["fwd_hbm_gbs"] = moved / (fwd_ms * 1e-3) / 1e9
            entry["fwd_frac_of_measured_hbm"] = entry["fwd_hbm_gbs"] / hbm_peak
            if backward:
                moved = sum(hbm_bytes(k, count, s, d) for k in ("sdpa", "delta", "sdpa_bwd_q", "sdpa_bwd_kv"))
                entry["fwd_bwd_hbm_gbs"] = moved / (entry["fwd_bwd_ms"] * 1e-3) / 1e9
                entry["fwd_bwd_frac_of_measured_hbm"] = entry["fwd_bwd_hbm_gbs"] / hbm_peak
            entry["hbm_bytes_per_launch"] = {k: hbm_bytes(k, count, s, d) for k in ("sdpa", "delta", "sdpa_bwd_q", "sdpa_bwd_kv")}
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


def decode_cases(args, world: int, torch, device, barrier, max_over_ranks) -> dict:
    """The step of a kv cache (one query row against every key so far), which is not a BASELINE configuration but
    is the other shape the ops are called in: bound by reading K and V once, so reported against the measured copy
    bandwidth. Values are random; parity of the shape is tests/test_sdpa_gpu.py's business."""
    from limn_b200._lib import lib

    L = lib()
    peak, _ = peaks()
    hbm_peak = float(peak.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    found = {}
    for name, bh_all, t_k, d in (("one_row_4096_keys_d128", 256, 4096, 128), ("one_row_2048_keys_d64", 1024, 2048, 64)):
        bh = bh_all // world
        q = torch.randn((bh, 1, d), device=device).to(torch.bfloat16)
        k, v = (torch.randn((bh, t_k, d), device=device).to(torch.bfloat16) for _ in range(2))
        out = torch.empty_like(q)
        lse = torch.empty((bh, 1), dtype=torch.float32, device=device)
        torch.cuda.synchronize()

        def launch():
            code = L.limn_b200_sdpa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, out.data_ptr(), lse.data_ptr(), 2, bh, 1, t_k, d, d, 0, d ** -0.5, None)
            if code:
                raise RuntimeError(L.limn_b200_last_error().decode())

        for _ in range(3):
            launch()
        trials = []
        for _ in range(3):
            barrier()
            time.sleep(args.rest_seconds)
            barrier()
            trials.append(max_over_ranks(timed(None, 20, launch)) / 20)
        ms = min(trials)
        moved = bh * (2 * t_k * d * 2 + 2 * d * 2 + 4)
        found[name] = {"problems_per_rank": bh, "ms": ms, "hbm_gbs": moved / (ms * 1e-3) / 1e9, "frac_of_measured_hbm": moved / (ms * 1e-3) / 1e9 / hbm_peak,
                       "bytes_per_launch": moved}
    return found


def off_grid_cases(args, world: int, torch, device, barrier, max_over_ranks) -> dict:
    """Shapes outside the four BASELINE configurations that the ops are still called with, device-resident, forward and
    forward+backward (row dot as its own launch). "float32": float32 storage, computed at float32 on the CUDA cores
    (limn's numpy and c devices run BASELINE's first configuration this way, and a model kept in float32 calls the
    ops like this), against the float32 multiply-add rate of the part (SMs x 128 lanes x 2 x the maximum SM clock: a
    nominal figure, nothing measures it here). "narrow_heads": bfloat16 with head dims that are not 64 or 128, which
    run zero-padded in the tensor-core kernels; credited with the flops of the real head dim."""
    from limn_b200._lib import lib

    L = lib()
    props = torch.cuda.get_device_properties(device)
    fma_peak = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12
    found = {"float32": {"fp32_fma_tflops_nominal": fma_peak}, "narrow_heads": {}}
    cases = (("float32", "reference_cpu_case_B1_H2_S128_D32_causal", 2, 128, 32, True),
             ("float32", "gpt_layer_in_float32_B32_H8_S256_D64_causal", 256, 256, 64, True),
             ("float32", "B4_H16_S1024_D128_causal", 64, 1024, 128, True),
             ("narrow_heads", "bf16_B8_H16_S2048_D96_causal", 128, 2048, 96, True),
             ("narrow_heads", "bf16_B32_H8_S256_D32_causal", 256, 256, 32, True))
    for family, name, bh_all, s, d, causal in cases:
        bh = max(1, bh_all // world)
        f32 = family == "float32"
        code = 0 if f32 else 2
        q, k, v, do = (torch.randn((bh, s, d), device=device).to(torch.float32 if f32 else torch.bfloat16) for _ in range(4))
        out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
        lse, delta = (torch.empty((bh, s), dtype=torch.float32, device=device) for _ in range(2))
        tail = (code, bh, s, s, d, d, int(causal), d ** -0.5, None)

        def check(status):
            if status:
                raise RuntimeError(L.limn_b200_last_error().decode())

        def forward():
            check(L.limn_b200_sdpa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, out.data_ptr(), lse.data_ptr(), *tail))

        def step():
            forward()
            check(L.limn_b200_sdpa_delta(out.data_ptr(), do.data_ptr(), delta.data_ptr(), code, bh * s, d, None))
            check(L.limn_b200_sdpa_bwd_q(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(), None, dq.data_ptr(), *tail))
            check(L.limn_b200_sdpa_bwd_kv(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(), None, dk.data_ptr(), dv.data_ptr(), *tail))

        entry = {"problems_per_rank": bh}
        for key, body, credit in (("fwd", forward, 1.0), ("fwd_bwd", step, 3.5)):
            for _ in range(3):
                body()
            trials = []
            for _ in range(3):
                barrier()
                trials.append(max_over_ranks(timed(None, 10, body)) / 10)
            ms = min(trials)
            entry[key + "_ms"] = ms
            entry[key + "_tflops"] = credit * fwd_flops(bh * world, s, d, causal) / (ms * 1e-3) / 1e12
            if f32:
                executed = (1.0 if key == "fwd" else 4.5) * fwd_flops(bh, s, d, causal) / (ms * 1e-3) / 1e12
                entry[key + "_executed_frac_of_fp32_fma_nominal"] = executed / fma_peak
        found[family][name] = entry
    return found


def errors(got: np.ndarray, want: np.ndarray) -> dict:
    """Both measures of one comparison: the raw max-abs error and the reference checker's, relative to
    max(1, max |want|) (limn/sdpa.py:251-259)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    raw = float(np.abs(got - want).max())
    biggest = float(np.abs(want).max())
    return {"raw_max_abs": raw, "normalised": raw / max(1.0, biggest), "max_abs_want": biggest}


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
    tensor_peak = float(peak.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    sustained_peak = float(peak.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
    total_flops = fwd_flops(bh, s, d, causal) * (3.5 if backward else 1.0)

    # ---- device-resident throughput: K steps, the best of three trials, each the max over ranks ----
    for _ in range(max(args.warmup, 3)):
        shard.step()
    # Each burst trial starts from the same state: a pause first, so that the board's power averaging has let go
    # of the trial before (at 1 kW the power cap pulls the SM clock from 1.97 to about 1.6 GHz within some tens
    # of milliseconds of back-to-back launches; what happens then is the "sustained" entry's business).
    def rested() -> None:
        barrier()
        time.sleep(args.rest_seconds)
        barrier()

    trials = []
    if sampler:
        sampler.begin("timed")
    for _ in range(3):
        rested()
        shard.launches = 0
        trial_ms = timed(shard, args.steps, shard.step)
        barrier()
        trials.append(max_over_ranks(trial_ms))
    if sampler:
        sampler.end("timed")
    launches = shard.launches
    ms = min(trials)
    value = total_flops * args.steps / (ms * 1e-3) / 1e12

    # dominant kernel alone (the forward), for the roofline entry
    fwd_trials = []
    for _ in range(3):
        rested()
        fwd_trials.append(max_over_ranks(timed(shard, args.steps, shard.forward)) / args.steps)
    fwd_ms = min(fwd_trials)
    fwd_rate = fwd_flops(per_rank, s, d, causal) / (fwd_ms * 1e-3) / 1e12

    # ---- the same step for seconds on end: long enough for the power cap to set the clock ----
    sustained = None
    if args.sustain_seconds > 0:
        many = max(args.steps, int(args.sustain_seconds * 1e3 / (ms / args.steps)) + 1)
        barrier()
        if sampler:
            sampler.begin("sustained")
        long_ms = max_over_ranks(timed(shard, many, shard.step))
        if sampler:
            sampler.end("sustained")
        sustained = {"steps": many, "seconds": long_ms * 1e-3, "ms_per_step": long_ms / many,
                     "value": total_flops * many / (long_ms * 1e-3) / 1e12, "unit": "TFLOP/s"}
        sustained["pct_of_measured_sustained_peak"] = 100 * sustained["value"] / world / sustained_peak

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
    clocks = sampler.stop() if sampler else {}

    # ---- the one collective: the gather of the output shards ----
    # Reported beside the compute-only number, never inside it. The shard is computed in a few chunks, and each
    # chunk's all-gather runs on a side stream while the next chunk computes: outputs of finished problems are
    # final. What the gather cannot go below is NVLink: every rank receives (N-1)/N of the whole output.
    gathered = None
    worst_rank_parity = None
    if world > 1 and not backward:
        items = per_rank * ((s + 255) // 256)
        parts = max(1, min(4, items // 256))
        while per_rank % parts:
            parts -= 1
        n_c = per_rank // parts
        stage = torch.empty((parts, world, n_c, s, d), dtype=torch.int16, device=device)
        side = torch.cuda.Stream(device=device)
        main_stream = torch.cuda.current_stream(device)
        done = [torch.cuda.Event() for _ in range(parts)]

        def gathered_step() -> None:
            for c in range(parts):
                shard.forward_range(c * n_c, n_c)
                done[c].record(main_stream)
                side.wait_event(done[c])
                with torch.cuda.stream(side):
                    dist.all_gather_into_tensor(stage[c].view(torch.bfloat16), shard.out[c * n_c:(c + 1) * n_c].view(torch.bfloat16))
            main_stream.wait_stream(side)

        for _ in range(3):  # warms the communicator and its buffers too
            gathered_step()
        g_steps = max(3, min(args.steps, 10))
        g_trials = []
        for _ in range(3):
            barrier()
            g_trials.append(max_over_ranks(timed(shard, g_steps, gathered_step)) / g_steps)
        g_ms = min(g_trials)
        inbound = (world - 1) * per_rank * s * d * 2
        gathered = {"value": total_flops / (g_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": g_ms, "chunks": parts,
                    "inbound_bytes_per_rank": inbound, "nvlink_floor_ms": inbound / 770e9 * 1e3,
                    "note": "forward + all-gather of O to every rank, chunked, the gather of a chunk overlapping the next chunk's kernels; "
                            "floor = bytes every rank must receive / 770 GB/s measured peer bandwidth"}
        barrier()
        if rank == 0:
            # the assembled tensor: the first problem of every rank's shard against the CPU implementation
            forward = cpu_kernels()[0]
            worst_rank_parity = {"raw_max_abs": 0.0, "normalised": 0.0, "ranks_checked": world}
            for r in range(world):
                q, k, v, _ = problem_inputs(workload, r * per_rank)
                want_out, _ = forward(q, k, v, causal=causal, scale=d ** -0.5)
                got = stage[0, r, 0].cpu().numpy().view(BF16).astype(np.float32)
                e = errors(got, want_out.astype(np.float32))
                worst_rank_parity["raw_max_abs"] = max(worst_rank_parity["raw_max_abs"], e["raw_max_abs"])
                worst_rank_parity["normalised"] = max(worst_rank_parity["normalised"], e["normalised"])
        del stage

    others = other_workloads(args, workload, world, rank, torch, device, barrier, max_over_ranks) if args.others else None
    if others is not None:
        others["decode"] = decode_cases(args, world, torch, device, barrier, max_over_ranks)
        others.update(off_grid_cases(args, world, torch, device, barrier, max_over_ranks))

    status = runtime.device_status()
    if status:
        raise SystemExit(f"a kernel gave up on a bounded wait (status 0x{status:08x}); no number is reported")

    if rank == 0:
        # spot parity of the timed launch: problems spread over this shard against the CPU implementation, both
        # error measures (the full-size parity of every configuration is tests/test_full_size_gpu.py)
        forward = cpu_kernels()[0]
        shard.forward()
        torch.cuda.synchronize()
        checked = sorted({0, per_rank // 2, per_rank - 1})
        parity = {"problems": [first_problem + p for p in checked], "out": {"raw_max_abs": 0.0, "normalised": 0.0},
                  "lse": {"raw_max_abs": 0.0, "normalised": 0.0}, "tolerance": {"out": 2e-2, "lse": 1e-3},
                  "every_rank_first_problem_after_gather": worst_rank_parity}
        for p in checked:
            q, k, v, _ = problem_inputs(workload, first_problem + p)
            want_out, want_lse = forward(q, k, v, causal=causal, scale=d ** -0.5)
            for key, e in (("out", errors(shard.out[p].cpu().numpy().view(BF16).astype(np.float32), want_out.astype(np.float32))),
                           ("lse", errors(shard.lse[p].cpu().numpy(), want_lse[..., 0]))):
                parity[key] = {m: max(parity[key][m], e[m]) for m in ("raw_max_abs", "normalised")}

        limn_numbers = None
        if args.limn and world == 1:
            limn_numbers = limn_subprocess(workload)

        sample = cpu_sample_size(workload, 12.0)
        cpu_seconds, cpu_flops = cpu_pass(workload, list(range(sample)))
        traffic, traffic_note = forward_traffic(workload, per_rank)
        line = {
            "metric": METRIC,
            "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 operands, f32 accumulate", "data": "synthetic",
            "config": {"workload": workload, "describes": WORKLOADS[workload][-1], "pass": "fwd+bwd" if backward else "fwd",
                       "problems_per_rank": per_rank, "sharding": "(batch, head) problems split evenly over ranks, no data-path collective",
                       "l2": "inputs larger than L2" if per_rank * s * d * 2 * 3 > 126e6 else "inputs smaller than L2 (resident between steps)",
                       "trials": f"best of 3 trials of K steps, each trial the max over ranks and preceded by a {args.rest_seconds} s pause"},
            "trials_ms_per_step": [t / args.steps for t in trials],
            "pct_of_peak": {"of_measured_burst": 100 * value / world / tensor_peak, "of_nominal_2250": 100 * value / world / 2250.0},
            "sustained": sustained,
            "roofline": {"bound": "tensor", "kernel": "sdpa_fwd_kernel", "achieved": fwd_rate, "peak": tensor_peak, "unit": "TFLOP/s",
                         "frac": fwd_rate / tensor_peak, "peak_kind": f"{peak_kind} burst (kernel timed alone, best of 3 x {args.steps} launches back to back, inputs larger than L2)",
                         "traffic": traffic, "traffic_note": traffic_note, "algorithmic_bytes": hbm_bytes("sdpa", per_rank, s, d), "ms_per_launch": fwd_ms},
            "cpu_baseline": {"value": cpu_flops / cpu_seconds / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count() or 1, "kind": cpu_kernels()[3],
                             "sample": f"{sample} of {bh} (batch, head) problems, {cpu_seconds:.1f} s"},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": up * world, "d2h_bytes_per_step": down * world,
                    "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": launches * world,
            "clocks": clocks.get("timed"),
            "clocks_sustained": clocks.get("sustained"),
            "gathered": gathered,
            "parity": parity,
            "limn": limn_numbers,
            "others": others,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------- limn itself on the GPU


def gpt_step(limn, *, dim: int, heads: int, layers: int, ctx: int, vocab: int = 256, attention_dtype=None, cast_in_place: bool = False):
    """A byte-level GPT training step shaped like limn's examples/train_stories.py (pre-norm blocks of causal
    attention and a 4x MLP, learned positions, AdamW, the loss realised with the update), at a width of our
    choosing and with the attention operands optionally cast to a half-width dtype, which is what puts the
    layer on the tensor-core kernels. `cast_in_place` moves the two casts to where the data lies token-major (the
    projection's output before it is sliced into q, k, v; the attention's result after it is reshaped back), which is
    what lets limn_b200.frontend.read_views_in_place() hand the kernels the views themselves. Returns
    (step(tokens, targets) -> loss, parameters)."""
    from limn.nn import Embedding, LayerNorm, Linear, parameters
    from limn.optim import AdamW

    Tensor = limn.Tensor

    class Layer:
        def __init__(self):
            self.norm_attention, self.norm_mlp = LayerNorm(dim), LayerNorm(dim)
            self.to_qkv, self.to_out = Linear(dim, 3 * dim), Linear(dim, dim)
            self.widen, self.narrow = Linear(dim, 4 * dim), Linear(4 * dim, dim)

        def __call__(self, x):
            b, t, c = x.shape
            projected = self.to_qkv(self.norm_attention(x))
            if attention_dtype is not None and cast_in_place:
                projected = projected.cast(attention_dtype)
            q, k, v = projected.reshape(b, t, 3, heads, c // heads).permute(2, 0, 3, 1, 4)
            if attention_dtype is not None and not cast_in_place:
                q, k, v = q.cast(attention_dtype), k.cast(attention_dtype), v.cast(attention_dtype)
            mixed = q.attention(k, v, causal=True)
            if attention_dtype is not None and not cast_in_place:
                mixed = mixed.cast(limn.float32)
            mixed = mixed.permute(0, 2, 1, 3).reshape(b, t, c)
            if attention_dtype is not None and cast_in_place:
                mixed = mixed.cast(limn.float32)
            x = x + self.to_out(mixed)
            return x + self.narrow(self.widen(self.norm_mlp(x)).relu())

    class Model:
        def __init__(self):
            self.tokens, self.positions = Embedding(vocab, dim), Embedding(ctx, dim)
            self.layers = [Layer() for _ in range(layers)]
            self.norm, self.head = LayerNorm(dim), Linear(dim, vocab, bias=False)

        def __call__(self, tokens):
            x = self.tokens(tokens) + self.positions(Tensor.arange(ctx))
            for layer in self.layers:
                x = layer(x)
            return self.head(self.norm(x))

    model = Model()
    params = parameters(model)
    opt = AdamW(params, lr=1e-3)

    def step(tokens, targets):
        opt.zero_grad()
        logp = model(tokens).log_softmax(-1)
        hit = Tensor.arange(vocab).reshape(1, 1, vocab).eq(targets.reshape(*targets.shape, 1))
        loss = -(logp * hit).sum() / float(targets.numel)
        loss.backward()
        opt.step(loss)
        opt.zero_grad()
        return loss

    return step, params


def limn_arm(workload: str) -> None:
    """limn itself on cuda:0, in a process of its own: first as it ships (its NVRTC-compiled scalar kernels,
    limn/cuda_emit.py:921-1083 through limn/backend_cuda.py:352-361), then with limn_b200.install(). Everything goes
    through Tensor.attention, autograd, the scheduler and the plan executor, under limn's capture, and is timed as
    limn's own benchmark times (examples/bench_attention.py:29-43): wall clock around replays, each of which ends in
    the device's finish(), best of three trials. Prints one JSON line."""
    if not limn_on_path():
        print(json.dumps({"unavailable": "limn is not staged under baseline/_ref"}))
        return
    import limn
    import limn.device

    import limn_b200

    rng = np.random.default_rng(0)

    def replay_ms(step, args, reps: int) -> float:
        replayed = limn.capture(step)

        def once() -> float:
            for _ in range(3):
                replayed(*args)
            start = time.perf_counter()
            for _ in range(reps):
                replayed(*args)
            return (time.perf_counter() - start) / reps * 1e3

        return min(once() for _ in range(3))

    def attention_case(name: str, problems: int, reps: int) -> dict:
        b, h, s, d, causal, backward, mul, v_kind, _seed, _ = WORKLOADS[name]
        problems = min(problems, b * h)
        shape = (problems, s, d)
        data = [rng.standard_normal(shape).astype(np.float32) * m for m in (mul, mul, 1.0)]

        def forward(q, k, v):
            return q.attention(k, v, causal=causal).realize()

        def train(q, k, v):
            out = q.attention(k, v, causal=causal)
            grads = limn.grad((out * out).sum(), [q, k, v])
            limn.realize(*grads)
            return tuple(grads)

        entry = {"problems": problems, "of": b * h, "shape": [s, d], "causal": causal}
        args = tuple(limn.Tensor(a, dtype=limn.bfloat16) for a in data)
        ms = replay_ms(forward, args, reps)
        entry["fwd_ms"], entry["fwd_tflops"] = ms, fwd_flops(problems, s, d, causal) / (ms * 1e-3) / 1e12
        if backward or name == "prefill_4k":
            args = tuple(limn.Tensor(a, dtype=limn.bfloat16, requires_grad=True) for a in data)
            ms = replay_ms(train, args, reps)
            entry["fwd_bwd_ms"], entry["fwd_bwd_tflops"] = ms, 3.5 * fwd_flops(problems, s, d, causal) / (ms * 1e-3) / 1e12
        return entry

    def layer_case(reps: int) -> dict:
        """The attention of one gpt_layer-sized transformer layer as a model holds it: q, k, v are slices of one
        bfloat16 projection output (batch, t, 3 * heads * hd), the result goes back to (batch, t, heads * hd); forward
        plus the gradient with respect to the projection. What differs between the columns is what limn puts around
        the three kernels: copies of q, k, v and dO and the row-dot reduce, or nothing."""
        b, h, s, d, causal, *_ = WORKLOADS["gpt_layer"]
        data = (rng.standard_normal((b, s, 3 * h * d)).astype(np.float32)).astype(BF16)
        weight = rng.standard_normal((b, s, h * d)).astype(np.float32).astype(BF16)

        def step(x, w):
            q, k, v = x.reshape(b, s, 3, h, d).permute(2, 0, 3, 1, 4)
            y = q.attention(k, v, causal=causal).permute(0, 2, 1, 3).reshape(b, s, h * d)
            (g,) = limn.grad((y * w).sum(), [x])
            limn.realize(y, g)
            return y, g

        args = (limn.Tensor(data.astype(np.float32), dtype=limn.bfloat16, requires_grad=True), limn.Tensor(weight.astype(np.float32), dtype=limn.bfloat16))
        ms = replay_ms(step, args, reps)
        return {"ms": ms, "fwd_bwd_tflops": 3.5 * fwd_flops(b * h, s, d, causal) / (ms * 1e-3) / 1e12,
                "what": "attention of one layer from its projection output to its result and back, B=32 H=8 S=256 D=64 causal bf16"}

    def gpt_case(reps: int, cast_in_place: bool = False) -> dict:
        ctx, batch = 256, 32
        limn.set_seed(0)
        step, params = gpt_step(limn, dim=512, heads=8, layers=6, ctx=ctx, attention_dtype=limn.bfloat16, cast_in_place=cast_in_place)
        tokens = rng.integers(0, 256, size=(batch, ctx + 1)).astype(np.int32)
        args = (limn.Tensor(tokens[:, :-1]), limn.Tensor(tokens[:, 1:]))
        ms = replay_ms(step, args, reps)
        return {"ms_per_step": ms, "tokens_per_s": batch * ctx / (ms * 1e-3), "model": "6 layers, d_model 512, 8 heads x 64, context 256, batch 32, "
                "float32 model with bfloat16 attention operands, synthetic byte tokens, AdamW step included", "parameters": int(sum(p.numel for p in params))}

    from limn_b200 import frontend as patches

    found = {"timing": "wall clock around replays of a captured step, each ending in the device's finish(); best of 3 trials",
             "kernels_as_shipped": {}, "limn_b200_installed": {},
             "limn_b200_installed_and_frontend_patched": {"patches": "limn_b200.frontend.fuse_row_dot() and read_views_in_place(); the model casts where the "
                                                                     "data lies token-major (gpt_step cast_in_place)"}}
    for label, install in (("kernels_as_shipped", False), ("limn_b200_installed", True), ("limn_b200_installed_and_frontend_patched", True)):
        limn.device.set_device("cuda")
        if install:
            limn_b200.install(limn.device.active())
        patched = label.endswith("patched")
        undo = [patches.fuse_row_dot(), patches.read_views_in_place()] if patched else []
        try:
            # the main workload on a subset of its problems (limn's scalar kernels need seconds for all of them), the GPT
            # attention layer in full, and the whole 6-layer training step around it
            found[label][workload] = attention_case(workload, 16, 3)
            if workload != "gpt_layer":
                found[label]["gpt_layer"] = attention_case("gpt_layer", 256, 10)
            found[label]["gpt_layer_from_projection"] = layer_case(10)
            found[label]["gpt_train_step"] = gpt_case(5, cast_in_place=patched)
        except Exception as err:
            found[label]["error"] = f"{type(err).__name__}: {err}"[:300]
        finally:
            for restore in undo:
                restore()
            limn.device.set_device("numpy")
    print(json.dumps(found), flush=True)


def limn_subprocess(workload: str) -> dict:
    """Run limn_arm in a process of its own (limn binds the driver API itself) and return what it printed."""
    if not (STAGED_LIMN / "limn" / "sdpa.py").is_file():
        return {"unavailable": "limn is not staged under baseline/_ref"}
    try:
        done = subprocess.run([sys.executable, str(Path(__file__).resolve()), "--limn-arm", workload], capture_output=True, text=True, timeout=900)
        lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
        if done.returncode != 0 or not lines:
            return {"unavailable": f"limn arm exited {done.returncode}: {done.stderr[-300:]}"}
        return json.loads(lines[-1])
    except Exception as err:
        return {"unavailable": f"{type(err).__name__}: {err}"[:300]}


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


def profile_decode(args) -> None:
    """For profiler captures: the decode case of `others.decode` (256 problems, one query row, 4096 keys, D = 128),
    launched `--steps` times after one warm-up launch."""
    import torch

    from limn_b200 import runtime
    from limn_b200._lib import lib

    torch.cuda.set_device(0)
    runtime.set_device(0)
    L = lib()
    bh, t_k, d = 256, 4096, 128
    q = torch.randn((bh, 1, d), device="cuda").to(torch.bfloat16)
    k, v = (torch.randn((bh, t_k, d), device="cuda").to(torch.bfloat16) for _ in range(2))
    out, lse = torch.empty_like(q), torch.empty((bh, 1), dtype=torch.float32, device="cuda")
    for _ in range(1 + args.steps):
        code = L.limn_b200_sdpa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, out.data_ptr(), lse.data_ptr(), 2, bh, 1, t_k, d, d, 0, d ** -0.5, None)
        if code:
            raise SystemExit(L.limn_b200_last_error().decode())
    torch.cuda.synchronize()
    print(json.dumps({"profiled": "decode one_row_4096_keys_d128", "problems": bh, "device_status": runtime.device_status()}))


def profile_float32(args) -> None:
    """For profiler captures: the float32 case B=4 H=16 S=1024 D=128 causal of `others.float32` (forward, row dot, dQ,
    dK/dV on the tiled CUDA-core kernels), launched `--steps` times after one warm-up pass."""
    import torch

    from limn_b200 import runtime
    from limn_b200._lib import lib

    torch.cuda.set_device(0)
    runtime.set_device(0)
    L = lib()
    bh, s, d = 64, 1024, 128
    q, k, v, do = (torch.randn((bh, s, d), device="cuda") for _ in range(4))
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    lse, delta = (torch.empty((bh, s), dtype=torch.float32, device="cuda") for _ in range(2))
    tail = (0, bh, s, s, d, d, 1, d ** -0.5, None)
    for _ in range(1 + args.steps):
        codes = (L.limn_b200_sdpa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, out.data_ptr(), lse.data_ptr(), *tail),
                 L.limn_b200_sdpa_delta(out.data_ptr(), do.data_ptr(), delta.data_ptr(), 0, bh * s, d, None),
                 L.limn_b200_sdpa_bwd_q(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(), None, dq.data_ptr(), *tail),
                 L.limn_b200_sdpa_bwd_kv(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(), None, dk.data_ptr(), dv.data_ptr(), *tail))
        if any(codes):
            raise SystemExit(L.limn_b200_last_error().decode())
    torch.cuda.synchronize()
    print(json.dumps({"profiled": "float32 B4_H16_S1024_D128_causal", "problems": bh, "device_status": runtime.device_status()}))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("limn_b200", "reference"), default="limn_b200")
    parser.add_argument("--workload", choices=sorted(WORKLOADS), default=DEFAULT_WORKLOAD)
    parser.add_argument("--profile", type=int, default=0, metavar="N", help="launch the kernels over the first N problems and exit (for ncu)")
    parser.add_argument("--profile-decode", action="store_true", help="launch the decode case of others.decode and exit (for ncu)")
    parser.add_argument("--profile-float32", action="store_true", help="launch a float32 case of others.float32 and exit (for ncu)")
    parser.add_argument("--backward", action="store_true", help="with --profile: run the backward kernels even for a forward-only workload")
    parser.add_argument("--no-others", dest="others", action="store_false", help="time only the named workload")
    parser.add_argument("--rest-seconds", type=float, default=0.5, help="pause before each burst trial")
    parser.add_argument("--sustain-seconds", type=float, default=2.0, help="length of the long timed region (0 to skip it)")
    parser.add_argument("--no-limn", dest="limn", action="store_false", help="skip the runs of limn itself on the GPU")
    parser.add_argument("--limn-arm", default=None, metavar="WORKLOAD", help="run limn itself on cuda:0 (stock kernels, then ours) and print one JSON line")
    args = parser.parse_args()
    if args.limn_arm:
        limn_arm(args.limn_arm)
    elif args.profile_decode:
        profile_decode(args)
    elif args.profile_float32:
        profile_float32(args)
    elif args.profile:
        profile_case(args)
    elif args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
