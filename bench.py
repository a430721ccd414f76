"""Benchmark of the triangle-attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg5|cfg3] [--impl ours|reference|reference-gpu]

One "step" is one forward + backward call of starting-node triangle attention on
synthetic inputs of the named BASELINE configuration (bf16, H=4, D=32, shared
bias, all-ones mask).  With N > 1 (launched by torchrun, one rank per GPU) the
pair rows are sharded across ranks; each step then also all-gathers the bias
shards and reduce-scatters the bias gradient (strong scaling: the total work is
fixed).  Rank 0 prints one JSON line.

`value` is the device-resident rate; `e2e` is the same step through the public
Python call with pinned host buffers: every input goes host -> device and every
result (out, dq, dk, dv, dbias) device -> host inside the timed region, streamed
in blocks of pair rows (rows are independent) so that the copies of neighbouring
blocks run under a block's kernels.

`--impl reference` times the reference's own CPU math (the oracle restatement of
its PyTorch `_reference`) on the host cores, on a bounded sample of rows of the
same configuration.  `--impl reference-gpu` times the reference's own operator
(its Triton kernels, from an offline install under baseline/_ref) on the same GPU
when that install is present; it is a reported comparison, never part of the
product path.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

WORKLOADS = {
    # name: (N, heads, head_dim) -- BASELINE configs 5 and 3
    "cfg5": dict(n=2048, heads=4, dim=32, label="config 5: starting node, bf16, fwd+bwd, B=1, N=2048, H=4, D=32"),
    "cfg3": dict(n=768, heads=4, dim=32, label="config 3: starting node, bf16, fwd+bwd, B=1, N=768, H=4, D=32"),
    # the remaining BASELINE configurations: timed device-resident on one GPU, short line (no roofline / e2e legs)
    "cfg1": dict(n=64, heads=4, dim=32, label="config 1: starting node, f32, fwd+bwd, B=1, N=64, H=4, D=32"),
    "cfg2": dict(n=384, heads=4, dim=32, label="config 2: starting node, bf16, fwd only, B=1, N=384 (350 valid), H=4, D=32"),
    "cfg4": dict(n=1024, heads=4, dim=32, label="config 4: ending node, bf16, fwd+bwd, ragged batch of 1024 and 700 tokens, H=4, D=32"),
}
FALLBACK_PEAK_TFLOPS = 1590.0
METRIC = "triangle_attention_fwd_bwd_tflops"


def flops(rows: int, cols: int, heads: int, dim: int, backward: bool) -> float:
    return float(rows) * heads * cols * cols * dim * (14.0 if backward else 4.0)


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            return float(data["bf16_tflops"]), float(data.get("bf16_tflops_sustained", data["bf16_tflops"])), "measured"
        except Exception:  # noqa: BLE001
            pass
    return FALLBACK_PEAK_TFLOPS, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs (read-only)."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self._nvml = None

    def _run(self):
        nvml = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(nvml.nvmlDeviceGetClockInfo(self._handle, nvml.NVML_CLOCK_SM))
                bits = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def make_inputs(n, heads, dim, row_lo, row_hi, seed, bias_rows=None):
    """Synthetic inputs of the configuration for rows [row_lo, row_hi): N(0,1)*0.5 q/k/v, N(0,1) bias and upstream.
    `bias_rows` query rows of the bias are made (default: as many as pair rows, the rank's shard of a square bias)."""
    gen = torch.Generator().manual_seed(seed)
    rows = row_hi - row_lo
    q, k, v = ((torch.randn(1, rows, n, heads, dim, generator=gen) * 0.5).to(torch.bfloat16) for _ in range(3))
    upstream = torch.randn(1, rows, n, heads, dim, generator=gen).to(torch.bfloat16)
    bias_shard = torch.randn(1, 1, heads, bias_rows or rows, n, generator=gen).to(torch.bfloat16)  # the rank's query rows
    mask = torch.ones(1, rows, n, dtype=torch.bool)
    return q, k, v, upstream, bias_shard, mask


# ----------------------------------------------------------------------------------------------
# reference arms
# ----------------------------------------------------------------------------------------------


class CpuOracle:
    """The oracle's forward+backward on a bounded sample of pair rows (rows are independent), timed on the host."""

    def __init__(self, n, heads, dim, budget_s, threads):
        from oracle import triangle_oracle as oracle

        self.oracle, self.n, self.heads, self.dim = oracle, n, heads, dim
        torch.set_num_threads(threads)
        self.gen = torch.Generator().manual_seed(1)
        self.bias = torch.randn(1, 1, heads, n, n, generator=self.gen)
        self._make(2)
        self.run()  # warm-up
        self._make(min(n, 16))
        per_row = self.run() / self.rows  # rate at a size that no longer fits the caches
        self._make(int(max(2, min(n, budget_s / max(per_row, 1e-6)))))

    def _make(self, rows):
        n, heads, dim = self.n, self.heads, self.dim
        self.rows = rows
        self.inputs = [torch.randn(1, rows, n, heads, dim, generator=self.gen) * 0.5 for _ in range(4)]
        self.mask = torch.ones(1, rows, n, dtype=torch.bool)

    def run(self):
        q, k, v, up = self.inputs
        t0 = time.perf_counter()
        self.oracle.forward_backward(q, k, v, self.mask, self.bias, up, budget_bytes=1 << 30)
        return time.perf_counter() - t0

    def rate(self):
        seconds = self.run()
        return flops(self.rows, self.n, self.heads, self.dim, True) / seconds / 1e12, self.rows, seconds


def cpu_oracle_rate(n, heads, dim, budget_s, threads):
    """One timed pass; returns (TFLOP/s, rows, seconds)."""
    return CpuOracle(n, heads, dim, budget_s, threads).rate()


def reference_arm(args, work):
    """The reference's CPU math on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n, heads, dim = work["n"], work["heads"], work["dim"]
    threads = os.cpu_count() or 1
    # a step is a bounded sample of rows sized so that the whole run stays near two minutes
    budget = max(1.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    cpu = CpuOracle(n, heads, dim, budget, threads)
    for _ in range(args.warmup):
        cpu.run()
    rates, rows_used, secs = [], 0, []
    for _ in range(args.steps):
        rate, rows_used, seconds = cpu.rate()
        rates.append(rate)
        secs.append(seconds)
    value = statistics.mean(rates)
    sample = f"{rows_used} of {n} rows per step (rows are independent), f32, all host threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * statistics.mean(secs), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": work["label"], "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def reference_gpu_arm(args, work):
    """The reference's own operator (Triton kernels) on this GPU, from the offline install under baseline/_ref.

    The install needs two modules that are not in this image: DanLing (only its container type is imported; dense
    inputs never touch it) and the version file the reference's build generates; both are stood in for by empty
    module objects.  Any failure prints an `unavailable` line and exits 0."""
    if int(os.environ.get("RANK", "0")) != 0:
        return

    def unavailable(why):
        print(json.dumps({"impl": "reference-gpu", "unavailable": " ".join(str(why).split())[:300]}), flush=True)

    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "oops").is_dir():
        return unavailable("baseline/_ref holds no install of the reference")
    if not torch.cuda.is_available():
        return unavailable("no GPU")
    try:
        import types

        sys.path.insert(0, str(ref_root))
        danling, tensors = types.ModuleType("danling"), types.ModuleType("danling.tensors")
        tensors.NestedTensor = type("NestedTensor", (), {})
        danling.tensors = tensors
        sys.modules.setdefault("danling", danling)
        sys.modules.setdefault("danling.tensors", tensors)
        version = types.ModuleType("oops._version")
        version.__version__ = version.version = "0.0.0"
        sys.modules.setdefault("oops._version", version)
        import oops  # the reference package

        n, heads, dim = work["n"], work["heads"], work["dim"]
        device = torch.device("cuda", 0)
        q, k, v, upstream, bias_shard, mask = (t.to(device) for t in make_inputs(n, heads, dim, 0, n, seed=100))
        q, k, v, bias = (t.requires_grad_(True) for t in (q, k, v, bias_shard))

        def step():
            out = oops.triangle_attention(q, k, v, mask, bias)
            return torch.autograd.grad(out, (q, k, v, bias), upstream)

        for _ in range(max(3, args.warmup)):
            step()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / args.steps
        with torch.no_grad():
            for _ in range(3):
                oops.triangle_attention(q, k, v, mask, bias)
            start.record()
            for _ in range(args.steps):
                oops.triangle_attention(q, k, v, mask, bias)
            stop.record()
            torch.cuda.synchronize()
            ms_fwd = start.elapsed_time(stop) / args.steps
        value = flops(n, n, heads, dim, True) / (ms * 1e-3) / 1e12
        line = {
            "impl": "reference-gpu", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": work["label"], "kernels": "the reference's Triton kernels, stock tile tables"},
            "fwd": {"ms": ms_fwd, "tflops": flops(n, n, heads, dim, False) / (ms_fwd * 1e-3) / 1e12},
        }
        print(json.dumps(line), flush=True)
    except Exception as error:  # noqa: BLE001
        unavailable(f"{type(error).__name__}: {error}")


# ----------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------


class StreamedStep:
    """One training step through the public call with host buffers, streamed in blocks of pair rows.

    Inputs live in pinned host memory; every block's q, k, v and upstream gradient are copied in on one stream, its
    forward + backward run on the compute stream, and its out, dq, dk, dv are copied back on a third stream, so that
    the copies of blocks i+1 and i-1 run under the kernels of block i.  The (sharded) bias goes in once per step; the
    bias gradient is summed over the blocks in f32 on the device and comes back once.  One copy per tensor block."""

    def __init__(self, host, device, run_block, blocks):
        self.device, self.run_block = device, run_block
        self.q, self.k, self.v, self.up, self.bias, self.mask = host
        rows = self.q.shape[1]
        self.blocks = [(i * rows // blocks, (i + 1) * rows // blocks) for i in range(blocks)]
        self.out = [torch.empty_like(self.q).pin_memory() for _ in range(4)]  # out, dq, dk, dv
        self.dbias = torch.empty_like(self.bias).pin_memory()
        self.s_in, self.s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        block_rows = max(hi - lo for lo, hi in self.blocks)
        shape = (1, block_rows, *self.q.shape[2:])
        self.staging = [[torch.empty(shape, dtype=self.q.dtype, device=device) for _ in range(4)] for _ in range(2)]
        self.mask_dev = self.mask.to(device)
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in (self.q, self.k, self.v, self.up, self.bias))
        self.d2h_bytes = sum(t.numel() * t.element_size() for t in (*self.out, self.dbias))

    def __call__(self):
        main = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(main)
        self.s_out.wait_stream(main)
        with torch.cuda.stream(self.s_in):
            bias = self.bias.to(self.device, non_blocking=True)
        free = [None, None]  # per staging set: the event after which it may be overwritten
        dbias_sum, keep = None, []
        for index, (lo, hi) in enumerate(self.blocks):
            stage = self.staging[index & 1]
            with torch.cuda.stream(self.s_in):
                if free[index & 1] is not None:
                    self.s_in.wait_event(free[index & 1])
                for dst, src in zip(stage, (self.q, self.k, self.v, self.up)):
                    dst[:, : hi - lo].copy_(src[:, lo:hi], non_blocking=True)
                arrived = self.s_in.record_event()
            main.wait_event(arrived)
            q, k, v, up = (t[:, : hi - lo] for t in stage)
            results = self.run_block(q, k, v, bias, self.mask_dev[:, lo:hi], up)  # (out, dq, dk, dv, dbias)
            dbias_sum = results[4].float() if dbias_sum is None else dbias_sum.add_(results[4])
            done = main.record_event()
            free[index & 1] = done
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for dst, src in zip(self.out, results[:4]):
                    dst[:, lo:hi].copy_(src, non_blocking=True)
            keep.append(results)  # the blocks' results stay alive until the copies have been issued and waited for
        final = dbias_sum.to(self.bias.dtype)
        self.s_out.wait_stream(main)
        with torch.cuda.stream(self.s_out):
            self.dbias.copy_(final, non_blocking=True)
        main.wait_stream(self.s_out)
        main.wait_stream(self.s_in)
        self._keep = (keep, final, bias)


def small_workload(args, work):
    """Configurations 1, 2 and 4: device-resident forward and forward+backward times on one GPU."""
    from oops_b200 import NestedTensor, triangle_attention
    from oops_b200.runtime import cabi

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    heads, dim, n = work["heads"], work["dim"], work["n"]
    gen = torch.Generator().manual_seed(0)
    name = args.workload
    if name == "cfg4":
        lengths = (1024, 700)
        stored = {k: [(torch.randn(L, L, heads, dim, generator=gen) * 0.5).to(torch.bfloat16) for L in lengths] for k in "qkv"}
        biases = [torch.randn(1, heads, L, L, generator=gen).to(torch.bfloat16) for L in lengths]
        tokens = [torch.rand(L, generator=gen) > 0.1 for L in lengths]
        masks = [tok[:, None] & tok[None, :] for tok in tokens]
        leaves, operands = [], []
        for k in "qkv":
            template = NestedTensor(stored[k], ragged_dims=(0, 1))
            values = template.concat.to(device).requires_grad_(True)
            leaves.append(values)
            operands.append(template.packed_like(values).transpose(-4, -3))
        mask_template = NestedTensor(masks, ragged_dims=(0, 1))
        operands.append(mask_template.packed_like(mask_template.concat.to(device)).transpose(-2, -1))
        bias_template = NestedTensor(biases, ragged_dims=(2, 3))
        bias_values = bias_template.concat.to(device).requires_grad_(True)
        leaves.append(bias_values)
        operands.append(bias_template.packed_like(bias_values).transpose(-2, -1))
        upstream = torch.randn(leaves[0].shape, generator=gen).to(torch.bfloat16).to(device)
        call = lambda: triangle_attention(*operands).concat  # noqa: E731
        scores = float(sum(L**3 for L in lengths)) * heads
        backward = True
    else:
        dtype = torch.float32 if name == "cfg1" else torch.bfloat16
        scale_in = 1.0 if name == "cfg1" else 0.5
        q, k, v = ((torch.randn(1, n, n, heads, dim, generator=gen) * scale_in).to(dtype).to(device).requires_grad_(True) for _ in range(3))
        bias = torch.randn(1, 1, heads, n, n, generator=gen).to(dtype).to(device).requires_grad_(True)
        upstream = torch.randn(1, n, n, heads, dim, generator=gen).to(dtype).to(device)
        valid = 350 if name == "cfg2" else n
        tok = torch.arange(n) < valid
        mask = (tok[:, None] & tok[None, :])[None].to(device)
        leaves = [q, k, v, bias]
        call = lambda: triangle_attention(q, k, v, mask, bias)  # noqa: E731
        scores = float(n) ** 3 * heads
        backward = name != "cfg2"

    def timed(fn, iters):
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / iters

    def step():
        out = call()
        if backward:
            torch.autograd.grad(out, leaves, upstream)

    iters = max(args.steps, 20)
    for _ in range(max(3, args.warmup)):
        step()
    before = cabi.launch_count()
    ms_step = timed(step, iters)
    launches = cabi.launch_count() - before
    with torch.no_grad():
        for _ in range(3):
            call()
        ms_fwd = timed(call, iters)
    peak, _, _ = measured_peak()
    total = scores * dim * (14.0 if backward else 4.0)
    status = cabi.device_status(reset=False)
    if status != 0:
        raise SystemExit(f"a kernel recorded device status {status}; the measurements above are void")
    line = {
        "metric": METRIC if backward else "triangle_attention_fwd_tflops", "value": total / (ms_step * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": 1, "steps": iters, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32" if name == "cfg1" else "bf16",
        "data": "synthetic", "config": {"workload": work["label"], "l2": "inputs fit in L2 at this size (no flush): a small-problem latency figure"
                                        if name in ("cfg1", "cfg2") else "inputs larger than L2 (no flush needed)"},
        "fwd": {"ms": ms_fwd, "tflops": scores * dim * 4.0 / (ms_fwd * 1e-3) / 1e12},
        "frac_of_bf16_peak": total / (ms_step * 1e-3) / 1e12 / peak, "gpu_launches": int(launches),
    }
    print(json.dumps(line), flush=True)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--workload", choices=sorted(WORKLOADS), default="cfg5")
    parser.add_argument("--impl", choices=("ours", "reference", "reference-gpu"), default="ours")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-extra", action="store_true", help="skip the secondary N=768 measurement")
    parser.add_argument("--rows", type=int, default=0,
                        help="time only the first ROWS pair rows of each GPU's shard (a slice for profiler captures; "
                             "rows are independent, FLOPs are counted for the slice)")
    parser.add_argument("--with-reference-gpu", action="store_true",
                        help="also time the reference's own GPU operator (a child process) and report it beside ours")
    args = parser.parse_args()
    work = WORKLOADS[args.workload]
    if args.impl == "reference":
        reference_arm(args, work)
        return
    if args.impl == "reference-gpu":
        reference_gpu_arm(args, work)
        return
    if args.workload in ("cfg1", "cfg2", "cfg4"):
        if args.gpus != 1:
            raise SystemExit("configurations 1, 2 and 4 are single-GPU workloads")
        small_workload(args, work)
        return

    import torch.distributed as dist

    from oops_b200 import triangle_attention
    from oops_b200.distributed.row_shard import gather_bias, row_sharded_triangle_attention, shard_bounds
    from oops_b200.runtime import cabi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run); got {world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU (there is no CPU fallback)")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    distributed = world > 1
    if distributed:
        dist.init_process_group("nccl", device_id=device)
    cabi.library()

    n, heads, dim = work["n"], work["heads"], work["dim"]
    lo, hi = shard_bounds(n, world, rank)
    if args.rows:
        hi = min(hi, lo + args.rows)
    total_rows = (hi - lo) * world

    def step(q, k, v, bias_shard, mask, upstream):
        if distributed:
            out = row_sharded_triangle_attention(q, k, v, mask, bias_shard)
        else:
            out = triangle_attention(q, k, v, mask, bias_shard)
        return (out, *torch.autograd.grad(out, (q, k, v, bias_shard), upstream))

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, iters):
        """Milliseconds per iteration, CUDA events on the current stream, max over ranks."""
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            fn()
        stop.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(stop) / iters], device=device)
        if distributed:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- N > 1: the sharded call against the unsharded one on a small problem, before anything is timed ------
    parity = None
    if distributed:
        n0 = 256
        full = [t.to(device) for t in make_inputs(n0, heads, dim, 0, n0, seed=5)]  # every rank builds the same problem
        fq, fk, fv, fup, fbias, fmask = full
        leaves = [t.detach().requires_grad_(True) for t in (fq, fk, fv, fbias)]
        whole = triangle_attention(leaves[0], leaves[1], leaves[2], fmask, leaves[3])
        whole_grads = torch.autograd.grad(whole, leaves, fup)
        a, b = shard_bounds(n0, world, rank)
        mine = [t[:, a:b].detach().requires_grad_(True) for t in (fq, fk, fv)]
        shard = fbias[:, :, :, a:b].detach().requires_grad_(True)
        part = row_sharded_triangle_attention(mine[0], mine[1], mine[2], fmask[:, a:b], shard)
        part_grads = torch.autograd.grad(part, (*mine, shard), fup[:, a:b])
        errors = [float((part.detach().float() - whole.detach()[:, a:b].float()).abs().max())]
        errors += [float((g.float() - w[:, a:b].float()).abs().max()) for g, w in zip(part_grads[:3], whole_grads[:3])]
        errors.append(float((part_grads[3].float() - whole_grads[3][:, :, :, a:b].float()).abs().max()))
        worst = torch.tensor(errors, device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        bound = 2e-2 * max(1.0, float(whole_grads[3].float().abs().max()))
        parity = {"problem": f"N={n0}, {world} row shards against the unsharded call (max-abs, max over ranks)",
                  "out": worst[0].item(), "dq": worst[1].item(), "dk": worst[2].item(), "dv": worst[3].item(),
                  "dbias_shard": worst[4].item(), "dbias_bound": bound}
        if max(parity["out"], parity["dq"], parity["dk"], parity["dv"]) != 0.0 or parity["dbias_shard"] > bound:
            raise SystemExit(f"row-sharded results differ from the unsharded call: {parity}")
        del full, leaves, whole, whole_grads, mine, shard, part, part_grads

    host = [t.pin_memory() for t in make_inputs(n, heads, dim, lo, hi, seed=100 + rank, bias_rows=n // world)]
    q, k, v, upstream, bias_shard, mask = (t.to(device) for t in host)
    q, k, v, bias_shard = (t.requires_grad_(True) for t in (q, k, v, bias_shard))

    # ---- device-resident throughput --------------------------------------------------------
    for _ in range(args.warmup):
        step(q, k, v, bias_shard, mask, upstream)
    launches_before = cabi.launch_count()
    with ClockSampler(local_rank) as clocks:
        ms_step = timed(lambda: step(q, k, v, bias_shard, mask, upstream), args.steps)
    launches = torch.tensor([cabi.launch_count() - launches_before], device=device, dtype=torch.int64)
    if distributed:
        dist.all_reduce(launches)
    total_flops = flops(total_rows, n, heads, dim, True)
    value = total_flops / (ms_step * 1e-3) / 1e12

    # ---- end to end: every input in from pinned host memory, every result out, every step ----
    def run_block(bq, bk, bv, bbias, bmask, bup):
        leaves = [t.detach().requires_grad_(True) for t in (bq, bk, bv, bbias)]
        return step(leaves[0], leaves[1], leaves[2], leaves[3], bmask, bup)

    streamed = StreamedStep(host, device, run_block, blocks=max(1, min(8, (hi - lo) // 64)))
    e2e_iters = max(2, min(args.steps, 5))
    streamed()
    ms_e2e = timed(streamed, e2e_iters)
    e2e_value = total_flops / (ms_e2e * 1e-3) / 1e12
    # the host link on its own: the step's copies without any kernel, one direction at a time and both at once
    def copies(inbound, outbound):
        def run():
            main_stream = torch.cuda.current_stream(device)
            streamed.s_in.wait_stream(main_stream)
            streamed.s_out.wait_stream(main_stream)
            if inbound:
                with torch.cuda.stream(streamed.s_in):
                    for dst, src in zip(link_in, (streamed.q, streamed.k, streamed.v, streamed.up)):
                        dst.copy_(src, non_blocking=True)
            if outbound:
                with torch.cuda.stream(streamed.s_out):
                    for dst, src in zip(streamed.out, link_in):
                        dst.copy_(src, non_blocking=True)
            main_stream.wait_stream(streamed.s_in)
            main_stream.wait_stream(streamed.s_out)
        return run

    link_in = [torch.empty(streamed.q.shape, dtype=streamed.q.dtype, device=device) for _ in range(4)]
    link = {name: timed(copies(*flags), 2) for name, flags in (("h2d_only_ms", (True, False)), ("d2h_only_ms", (False, True)),
                                                                ("both_directions_ms", (True, True)))}
    del link_in
    e2e = {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": streamed.h2d_bytes * world,
           "host_link": link,
           "d2h_bytes_per_step": streamed.d2h_bytes * world, "row_blocks": len(streamed.blocks),
           "results_copied_back": ["out", "dq", "dk", "dv", "dbias"]}
    del streamed

    # ---- the tensor kernels one by one -----------------------------------------------------------------
    peak, peak_sustained, peak_kind = measured_peak()
    with torch.no_grad():
        bias_full = gather_bias(bias_shard.detach()) if distributed else bias_shard.detach()
        fwd = lambda: triangle_attention(q.detach(), k.detach(), v.detach(), mask, bias_full)  # noqa: E731
        for _ in range(3):
            fwd()
        before = cabi.launch_count()
        ms_fwd = timed(fwd, args.steps)
        fwd_launches = (cabi.launch_count() - before) // args.steps
    fwd_flops_rank = flops(hi - lo, n, heads, dim, False)
    fwd_tflops = fwd_flops_rank / (ms_fwd * 1e-3) / 1e12
    # dQ, dK and dV together take the single-pass kernel (five products); the bias gradient its own (two).  A call
    # also launches the row-dot kernel (and, for rows split into groups, the two partial-plane adds), a few percent
    # of the group, so a group's rate slightly understates its tensor kernel.
    unit = flops(hi - lo, n, heads, dim, False) / 2.0  # one C x C x D product over this rank's rows
    groups = {}
    for name, wanted, products in (("dqkv", "qkv", 5), ("dbias", "b", 2)):
        ql, kl, vl, bl = (t.detach().requires_grad_(c in wanted) for t, c in ((q, "q"), (k, "k"), (v, "v"), (bias_full, "b")))
        out_l = triangle_attention(ql, kl, vl, mask, bl)
        targets = [t for t in (ql, kl, vl, bl) if t.requires_grad]
        run = lambda: torch.autograd.grad(out_l, targets, upstream, retain_graph=True)  # noqa: E731
        for _ in range(2):
            run()
        before = cabi.launch_count()
        ms = timed(run, args.steps)
        rate = products * unit / (ms * 1e-3) / 1e12
        groups[name] = {"ms": ms, "tflops_per_gpu": rate, "frac_of_bf16_peak": rate / peak,
                        "launches": (cabi.launch_count() - before) // args.steps, "products": products}
        del out_l, targets, run, ql, kl, vl, bl

    profile = {}
    traffic_file = ROOT / "profiles" / "traffic.json"
    if traffic_file.exists():
        try:
            profile = json.loads(traffic_file.read_text())
        except Exception:  # noqa: BLE001
            profile = {}

    def traffic(kernel):
        per_row = profile.get("%s_dram_bytes_per_row_n%d" % (kernel, n))
        return None if per_row is None else per_row * (hi - lo)

    # the kernel with the largest share of a training step (ncu launch list): the single-pass dQ/dK/dV kernel
    roofline = {
        "bound": "tensor", "kernel": "ta_bwd_fused_kernel (timed as the dQ+dK+dV reverse call: %d launches, the helper "
        "kernels a few percent of it)" % groups["dqkv"]["launches"],
        "achieved": groups["dqkv"]["tflops_per_gpu"], "peak": peak, "unit": "TFLOP/s",
        "frac": groups["dqkv"]["frac_of_bf16_peak"], "peak_kind": peak_kind, "ms": groups["dqkv"]["ms"],
        "traffic": traffic("dqkv"),
        "forward": {"kernel": "ta_fwd_kernel (one call; %d launch(es))" % fwd_launches, "achieved": fwd_tflops,
                    "frac": fwd_tflops / peak, "ms": ms_fwd, "traffic": traffic("forward")},
        "dbias": dict(groups["dbias"], traffic=traffic("dbias")),
    }

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "workload": work["label"] + (f" (slice: {hi - lo} rows per GPU)" if args.rows else ""), "rows_per_gpu": hi - lo, "sharding": "pair rows; bias all-gather, dbias reduce-scatter"
            if distributed else "single GPU", "l2": "inputs larger than L2 (no flush needed)",
            "tensor_path": {"forward": None, "backward": None},
        },
        "frac_of_bf16_peak": value / (peak * world), "frac_of_bf16_sustained": value / (peak_sustained * world),
        "fwd": {"ms": ms_fwd, "tflops_per_gpu": fwd_tflops, "frac_of_bf16_peak": fwd_tflops / peak},
        "clocks": clocks.summary(),
        "e2e": e2e,
        "gpu_launches": int(launches.item()),
        "roofline": roofline,
    }
    if parity is not None:
        line["parity"] = parity
    probe = cabi.make_problem(q.detach(), k.detach(), v.detach(), mask, bias_full, dim**-0.5)
    line["config"]["tensor_path"] = {
        "forward": bool(cabi.library().oops_ta_uses_tensor_path(cabi.byref(probe), 0) == 1),
        "backward": bool(cabi.library().oops_ta_uses_tensor_path(cabi.byref(probe), 1) == 1),
    }

    # ---- secondary: BASELINE config 3 (N=768) on one GPU -------------------------------------
    if rank == 0 and not distributed and not args.no_extra and args.workload != "cfg3":
        n3 = WORKLOADS["cfg3"]["n"]
        del host
        t3 = [t.to(device) for t in make_inputs(n3, heads, dim, 0, n3, seed=7)]
        q3, k3, v3, up3, b3, m3 = t3
        q3, k3, v3, b3 = (t.requires_grad_(True) for t in (q3, k3, v3, b3))
        for _ in range(3):
            step(q3, k3, v3, b3, m3, up3)
        ms3 = timed(lambda: step(q3, k3, v3, b3, m3, up3), max(args.steps, 10))
        with torch.no_grad():
            ms3f = timed(lambda: triangle_attention(q3, k3, v3, m3, b3), max(args.steps, 10))
        f3, f3f = flops(n3, n3, heads, dim, True), flops(n3, n3, heads, dim, False)
        # the gate of the following output projection, fused into the forward epilogue or applied as its own pass
        from oops_b200 import triangle_attention_gated
        from oops_b200.attention.gate.gate_attention_output import _run_gate

        gate3 = torch.randn(q3.shape, dtype=q3.dtype, device=device)
        with torch.no_grad():
            fused = lambda: triangle_attention_gated(q3, k3, v3, gate3, m3, b3)  # noqa: E731

            def unfused():
                values = triangle_attention(q3, k3, v3, m3, b3)
                gated = torch.empty_like(values)
                _run_gate(values, gate3, gated)
                return gated

            for _ in range(3):
                fused(), unfused()
            ms_fused, ms_unfused = timed(fused, max(args.steps, 10)), timed(unfused, max(args.steps, 10))
        pass_bytes = q3.numel() * q3.element_size()
        gated_entry = {
            "fused_forward_ms": ms_fused, "forward_then_gate_kernel_ms": ms_unfused,
            "saved_hbm_bytes": 2 * pass_bytes,  # the attention values are neither written nor read back
            "note": "inference, N=768: sigmoid(gate) * attention in the forward kernel's epilogue against the forward "
                    "kernel followed by the library's element-wise gate kernel",
        }
        # the layer norm that precedes the projections, on a pair representation of 2048 x 2048 cells (128 channels, bf16,
        # f32 parameters): HBM-bound byte work, reported against the measured copy bandwidth
        from oops_b200 import layer_norm
        hbm_gbs = 6551.4
        try:
            hbm_gbs = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["hbm_gbs"])
        except Exception:  # noqa: BLE001
            pass
        ln_rows, ln_width = 2048 * 2048, 128  # the pair representation of config 5: 1.07 GB per tensor
        ln_x = torch.randn(ln_rows, ln_width, device=device, dtype=torch.bfloat16).requires_grad_(True)
        ln_w = torch.ones(ln_width, device=device).requires_grad_(True)
        ln_b = torch.zeros(ln_width, device=device).requires_grad_(True)
        ln_up = torch.randn(ln_rows, ln_width, device=device, dtype=torch.bfloat16)
        with torch.no_grad():
            ln_fwd = lambda: layer_norm(ln_x, ln_width, ln_w, ln_b)  # noqa: E731
            for _ in range(3):
                ln_fwd()
            ms_ln_f = timed(ln_fwd, max(args.steps, 10))
        ln_out = layer_norm(ln_x, ln_width, ln_w, ln_b)
        ln_bwd = lambda: torch.autograd.grad(ln_out, (ln_x, ln_w, ln_b), ln_up, retain_graph=True)  # noqa: E731
        for _ in range(3):
            ln_bwd()
        ms_ln_b = timed(ln_bwd, max(args.steps, 10))
        ln_bytes = ln_rows * ln_width * 2
        ln_entry = {
            "rows": ln_rows, "width": ln_width, "forward_ms": ms_ln_f, "forward_gbs": 2 * ln_bytes / ms_ln_f / 1e6,
            "forward_frac_of_hbm": 2 * ln_bytes / ms_ln_f / 1e6 / hbm_gbs, "backward_ms": ms_ln_b,
            "backward_gbs": 3 * ln_bytes / ms_ln_b / 1e6, "backward_frac_of_hbm": 3 * ln_bytes / ms_ln_b / 1e6 / hbm_gbs,
            "hbm_peak_gbs": hbm_gbs,
            "note": "algorithmic bytes: forward reads x and writes y, reverse reads dy and x and writes dx (row statistics "
                    "and parameter partials are below 2 % of that); inputs larger than L2",
        }
        del ln_x, ln_out, ln_up
        line["n768"] = {
            "layer_norm": ln_entry,
            "workload": WORKLOADS["cfg3"]["label"], "fwd_bwd_ms": ms3, "fwd_bwd_tflops": f3 / ms3 / 1e9,
            "fwd_bwd_frac_of_bf16_peak": f3 / ms3 / 1e9 / peak, "fwd_ms": ms3f, "fwd_tflops": f3f / ms3f / 1e9,
            "fwd_frac_of_bf16_peak": f3f / ms3f / 1e9 / peak, "gated_output": gated_entry,
        }

    # a kernel that gave up a bounded wait leaves undefined results: none may have
    status = cabi.device_status(reset=False)
    if status != 0:
        raise SystemExit(f"a kernel recorded device status {status}; the measurements above are void")

    # ---- CPU baseline: the oracle on the host cores, bounded sample, rank 0 at N=1 only ------
    if rank == 0 and not distributed and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        rate, rows_used, seconds = cpu_oracle_rate(n, heads, dim, 12.0, threads)
        line["cpu_baseline"] = {
            "value": rate, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{rows_used} of {n} rows (rows are independent), f32, {seconds:.1f} s",
        }
    # ---- optional: the reference's own operator on the same GPU, in a child process ----------
    if rank == 0 and not distributed and args.with_reference_gpu:
        child = subprocess.run(
            [sys.executable, str(Path(__file__).resolve()), "--impl", "reference-gpu", "--workload", args.workload,
             "--steps", str(max(3, min(args.steps, 10))), "--warmup", "3"], capture_output=True, text=True, timeout=900,
        )
        reported = [ln for ln in child.stdout.splitlines() if ln.startswith("{")]
        line["reference_gpu"] = json.loads(reported[-1]) if reported else {"unavailable": child.stderr[-300:]}
        if "value" in line["reference_gpu"]:
            line["reference_gpu"]["ours_over_reference"] = value / line["reference_gpu"]["value"]
    if rank == 0:
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
