#!/usr/bin/env python
"""Benchmark of the hot path: fused residual ADD + RMSNorm on tiled BF16 storage.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one pass of iomb_add_rmsnorm over one batch of synthetic input: 16
planes of the TinyLlama prefill shape (rows 8192, hidden 2048, BF16, eps 1e-5),
one launch, 2.1 GB of algorithmic traffic, so every step streams from HBM (the
batch is 17 times the L2 capacity). With N > 1 every rank runs the same batch on
its own GPU (row shards are independent: no data-path collective) and rank 0
prints the aggregate. One JSON line is printed; see the keys below.

`--impl reference` times the reference's own CPU backend (oracle/_ref when the
shim is built, else the plain-C oracle port) on the host cores.
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
for entry in (str(ROOT), str(ROOT / "tests")):
    if entry not in sys.path:
        sys.path.insert(0, entry)

PLANES, ROWS, HIDDEN, EPS = 16, 8192, 2048, 1e-5
ELEM = 2
ELEMENTS = PLANES * ROWS * HIDDEN
# x and residual read, rounded sum and normalised output written, scale read once
ALGORITHMIC_BYTES = 4 * ELEMENTS * ELEM + HIDDEN * ELEM
METRIC = "achieved HBM GB/s, fused residual ADD + RMSNorm (BF16, TinyLlama prefill shape)"
WORKLOAD = (f"C2 x{PLANES}: BF16 [{PLANES},{ROWS},{HIDDEN}] residual ADD + RMSNorm, eps 1e-5, "
            "x,r ~ N(0,1), w ~ N(1,0.02)")
# dram__bytes_read.sum + dram__bytes_write.sum of one rmsnorm_kernel launch, from
# the ncu capture summarised in profiles/ (taken on a [2,8192,2048] case; traffic
# is proportional to the rows processed, so it is scaled by the plane count).
NCU_TRAFFIC_BYTES_PER_PLANE = 213.98e6 / 2     # 134.32 MB read + 79.66 MB written, 2 planes


def configure(planes: int) -> None:
    """Resizes the batch (the default is the benchmark's; profiler captures shrink it)."""
    global PLANES, ELEMENTS, ALGORITHMIC_BYTES, WORKLOAD
    PLANES = planes
    ELEMENTS = PLANES * ROWS * HIDDEN
    ALGORITHMIC_BYTES = 4 * ELEMENTS * ELEM + HIDDEN * ELEM
    WORKLOAD = (f"C2 x{PLANES}: BF16 [{PLANES},{ROWS},{HIDDEN}] residual ADD + RMSNorm, "
                "eps 1e-5, x,r ~ N(0,1), w ~ N(1,0.02)")


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during a timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(maxima),
                "reasons": sorted(reasons), "samples": len(clocks)}


def synthetic_inputs(seed: int):
    """Seeded logical payloads (BF16 codes) of the batch; C2's distributions."""
    import numpy as np

    def f32_to_bf16_bits(values):
        bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
        return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)

    rng = np.random.default_rng(seed)
    shape = (PLANES, ROWS, HIDDEN)
    x = f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32))
    r = f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32))
    w = f32_to_bf16_bits((1.0 + 0.02 * rng.standard_normal((1, HIDDEN))).astype(np.float32))
    return x, r, w


def run_ours(args) -> dict:
    import numpy as np
    import torch
    import torch.distributed as dist

    from iom_b200.device import DeviceMemoryConfig, make_b200_device
    from iom_b200.tensor import DataType, TensorSpec

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the B200 backend has no CPU fallback")
    torch.cuda.set_device(local_rank)
    # Libraries (NCCL's version banner) write to stdout; the one JSON line must be
    # the only thing there, so fd 1 points at stderr until the result is printed.
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    args._restore_stdout = lambda: (os.dup2(saved_stdout, 1), os.close(saved_stdout))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    arena = max(5 * PLANES * ROWS * HIDDEN * ELEM + 7 * ROWS * HIDDEN * ELEM + (64 << 20),
                0 if args.no_ops else 5 << 30)
    device = make_b200_device(local_rank, DeviceMemoryConfig(arena // 32 * 32))
    queue = device.create_ops()
    shape = (PLANES, ROWS, HIDDEN)
    spec = TensorSpec(shape, DataType.BF16)
    x, r, total, out = (device.create_tensor(spec) for _ in range(4))
    scale = device.create_tensor(TensorSpec((1, HIDDEN), DataType.BF16))
    logical_bytes = spec.logical_nbytes()
    staging = device.create_workspace(logical_bytes + 64)

    # Seeded inputs live in pinned host memory in the logical row-major layout the
    # reference's copy_from_host takes.
    x_host, r_host, w_host = synthetic_inputs(seed=1000 + rank)
    pinned = {}
    for name, array in (("x", x_host), ("r", r_host)):
        buffer = torch.empty(array.size, dtype=torch.int16, pin_memory=True)
        buffer.numpy().view(np.uint16)[:] = array.reshape(-1)
        pinned[name] = buffer
    out_host = torch.empty(ELEMENTS, dtype=torch.int16, pin_memory=True)
    scale.view().copy_from_host(w_host, staging.view())
    x.view().copy_from_host(pinned["x"].numpy(), staging.view())
    r.view().copy_from_host(pinned["r"].numpy(), staging.view())

    def step():
        token = queue.add_rmsnorm(x.view(), r.view(), scale.view(), total.view(), out.view(), EPS)
        if token <= 0:
            raise RuntimeError(f"add_rmsnorm rejected with oid {token}")
        return token

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput (`value`) -----------------------------
    for _ in range(args.warmup):
        token = step()
    queue.wait(token)
    barrier()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        start.record(queue.stream)
        for _ in range(args.steps):
            token = step()
        stop.record(queue.stream)
        queue.wait(token)
        barrier()
    elapsed_ms = start.elapsed_time(stop)
    clocks = sampler.summary()

    # ---- end to end through the public API with host buffers (`e2e`) -------
    e2e_steps = max(1, min(args.steps, 3))

    def e2e_step():
        x.view().copy_from_host(pinned["x"].numpy(), staging.view())
        r.view().copy_from_host(pinned["r"].numpy(), staging.view())
        queue.wait(step())
        out.view().copy_to_host(out_host.numpy(), staging.view())

    # The same step with the asynchronous transfer operations: the batch goes plane by
    # plane through two queues (streams), so that one queue's device-to-host copy
    # runs while the other's host-to-device copies do (both PCIe directions busy).
    plane_bytes = ROWS * HIDDEN * ELEM
    lanes = []

    def e2e_pipelined_step():
        if not lanes:
            for q in (queue, device.create_ops()):
                lanes.append((q, [device.create_workspace(plane_bytes + 64) for _ in range(3)]))
        tokens = [None, None]
        for plane in range(PLANES):
            q, (sx, sr, so) = lanes[plane % 2]
            chunk = slice(plane * ROWS * HIDDEN, (plane + 1) * ROWS * HIDDEN)
            xv, rv = x.view().select(0, plane), r.view().select(0, plane)
            tv, ov = total.view().select(0, plane), out.view().select(0, plane)
            for token in (q.upload(xv, pinned["x"].numpy()[chunk], sx.view()),
                          q.upload(rv, pinned["r"].numpy()[chunk], sr.view()),
                          q.add_rmsnorm(xv, rv, scale.view(), tv, ov, EPS)):
                if token <= 0:
                    raise RuntimeError(f"pipelined step rejected with oid {token}")
            tokens[plane % 2] = q.download(ov, out_host.numpy()[chunk], so.view())
            if tokens[plane % 2] <= 0:
                raise RuntimeError(f"download rejected with oid {tokens[plane % 2]}")
        for (q, _), token in zip(lanes, tokens):
            q.wait(token)

    e2e_ms = float("nan")
    e2e_sync_ms = float("nan")
    if not args.no_e2e:
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_sync_ms = (time.perf_counter() - t0) * 1e3
        reference_out = out_host.clone()
        out_host.zero_()
        e2e_pipelined_step()
        barrier()
        if not torch.equal(reference_out, out_host):
            raise RuntimeError("pipelined end-to-end step and synchronous step disagree")
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_pipelined_step()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3

    # ---- whole-tensor sum of squares across ranks (the one exchange step) ----
    sumsq_info = None
    if world > 1:
        from iom_b200.sharding import all_gather_sum
        scratch = device.create_workspace(int(device._lib.iomb_sumsq_scratch_bytes()))
        local = torch.zeros(1, dtype=torch.float32, device=device.torch_device)

        def sumsq_step():
            token = queue.sumsq(total.view(), scratch.view(), local.data_ptr())
            if token <= 0:
                raise RuntimeError(f"sumsq rejected with oid {token}")
            queue.wait(token)
            return all_gather_sum(local)

        combined = sumsq_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(5):
            combined = sumsq_step()
        torch.cuda.synchronize()
        sumsq_ms = (time.perf_counter() - t0) * 1e3 / 5
        gathered = [torch.empty_like(combined.reshape(1)) for _ in range(world)]
        dist.all_gather(gathered, combined.reshape(1))
        sumsq_info = {"value": float(combined), "ms": sumsq_ms,
                      "identical_on_all_ranks": all(torch.equal(gathered[0], g) for g in gathered),
                      "bytes_read_per_rank": ELEMENTS * ELEM,
                      "combine": "all_gather of one FP32 partial per rank, added in rank order"}
        scratch.close()

    table = None
    if world == 1 and not args.no_ops:
        for t in (x, r, total, out, scale):
            t.close()
        staging.close()
        table = ops_table(device, queue)

    times = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = (float(v) for v in times.tolist())

    result = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        per_launch_ms = elapsed_ms / args.steps
        achieved = ALGORITHMIC_BYTES / per_launch_ms / 1e6
        result = {
            "metric": METRIC,
            "value": world * ALGORITHMIC_BYTES * args.steps / elapsed_ms / 1e6,
            "unit": "GB/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": per_launch_ms,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f32 accumulate, bf16 storage",
            "data": "synthetic (seeded normal, the TinyLlama prefill configuration's distributions)",
            "config": {"workload": WORKLOAD, "launches_per_step": 1,
                       "algorithmic_bytes_per_step": ALGORITHMIC_BYTES,
                       "l2": f"inputs larger than L2 ({ALGORITHMIC_BYTES / 1e9:.2f} GB touched "
                             "per step, L2 is 126 MB)",
                       "order": "LANES16", "pct_of_8TBps": None},
            "clocks": clocks,
            "e2e": {"value": world * ALGORITHMIC_BYTES * e2e_steps / e2e_ms / 1e6, "unit": "GB/s",
                    "h2d_bytes_per_step": 2 * logical_bytes, "d2h_bytes_per_step": logical_bytes,
                    "steps": e2e_steps,
                    "path": "per plane, alternating over two queues: upload(x), upload(r), "
                            "add_rmsnorm, download(out); pinned host buffers in the logical layout",
                    "synchronous_value": world * ALGORITHMIC_BYTES * e2e_steps / e2e_sync_ms / 1e6,
                    "synchronous_path": "copy_from_host(x), copy_from_host(r), add_rmsnorm, "
                                        "copy_to_host(out)"},
            "gpu_launches": args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES_PER_PLANE * PLANES,
                         "peak_source": f"of {peak_kind}", "kernel": "rmsnorm_kernel<2,16,true>",
                         "algorithmic_bytes_per_launch": ALGORITHMIC_BYTES},
        }
        result["config"]["pct_of_8TBps"] = 100.0 * achieved / 8000.0
        if table is not None:
            result["ops"] = table
        if sumsq_info is not None:
            result["sumsq_across_ranks"] = sumsq_info
    queue.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result


# ---- per-operation table (supporting numbers beside the headline) ------------------

def ops_table(device, queue, only=None, iters: int = 10) -> dict:
    """Device-resident GB/s (algorithmic bytes / CUDA-event time) of every operation
    of the path on HBM-sized inputs, plus single-launch microseconds of the
    decode-step data movement. Inputs are random bytes reinterpreted per leaf:
    timing does not depend on the values."""
    import ctypes

    import torch

    from iom_b200.tensor import DataType, TensorSpec

    lib = device._lib
    made = []

    def tensor(shape, dtype, kind="normal"):
        t = device.create_tensor(TensorSpec(shape, dtype))
        n = t.storage_nbytes
        if dtype == DataType.BF16 and kind == "normal":
            t.storage().copy_(torch.randn(n // 2, device=device.torch_device)
                              .to(torch.bfloat16).view(torch.uint8))
        elif dtype == DataType.F32 and kind == "normal":
            t.storage().copy_(torch.randn(n // 4, device=device.torch_device).view(torch.uint8))
        else:
            t.storage().copy_(torch.randint(0, 64, (n,), device=device.torch_device,
                                            dtype=torch.uint8))
        made.append(t)
        return t

    def release():
        while made:
            made.pop().close()

    def timed(launch, inner=1):
        """Median CUDA-event time of one launch; `inner` launches share one event
        pair for microsecond-scale operations (the figure then includes the host's
        issue rate through this Python layer, as a caller would see it)."""
        torch.cuda.synchronize()    # input fills run on another stream: let them finish first
        for _ in range(3):
            token = launch()
        queue.wait(token)
        pairs = []
        for _ in range(iters):
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record(queue.stream)
            for _ in range(inner):
                token = launch()
            b.record(queue.stream)
            pairs.append((a, b))
            queue.wait(token)
        torch.cuda.synchronize()
        times = sorted(a.elapsed_time(b) for a, b in pairs)
        return times[len(times) // 2] / inner

    def ok(token):
        if token <= 0:
            raise RuntimeError(f"operation rejected with oid {token}")
        return token

    results = {}

    def record(name, nbytes, launch, shape, inner=1):
        if only is not None and name != only:
            return
        ms = timed(launch, inner)
        results[name] = {"GB/s": nbytes / ms / 1e6, "us": ms * 1e3, "bytes": nbytes,
                         "pct_of_8TBps": nbytes / ms / 1e6 / 80.0, "shape": shape}

    M, N = 131072, 2048          # 2^28 elements: far beyond L2
    E = M * N
    for dtype, name, b in ((DataType.BF16, "bf16", 2), (DataType.F32, "f32", 4),
                           (DataType.I32, "i32", 4)):
        wanted = [f"{op}_{name}_{form}" for op in ("add", "mul") for form in ("full", "row", "col")]
        if only is not None and only not in wanted:
            continue
        x, y, o = tensor((M, N), dtype), tensor((M, N), dtype), tensor((M, N), dtype)
        row, col = tensor((1, N), dtype), tensor((M, 1), dtype)
        fn = queue.mul if dtype == DataType.F32 else queue.add
        op = "mul" if dtype == DataType.F32 else "add"
        record(f"{op}_{name}_full", 3 * E * b, lambda: ok(fn(x.view(), y.view(), o.view())),
               f"[{M},{N}]")
        record(f"{op}_{name}_row", (2 * E + N) * b, lambda: ok(fn(x.view(), row.view(), o.view())),
               f"[{M},{N}] op [1,{N}]")
        record(f"{op}_{name}_col", (2 * E + M) * b, lambda: ok(fn(x.view(), col.view(), o.view())),
               f"[{M},{N}] op [{M},1]")
        release()
    # RMSNorm family, BF16
    for label, shape, eps in (("tinyllama", (16, 8192, 2048), 1e-5), ("c5shard", (32768, 8192), 1e-6)):
        names = [f"rmsnorm_{label}", f"add_rmsnorm_{label}", f"rmsnorm_sequential_{label}"]
        if only is not None and only not in names:
            continue
        cols = shape[-1]
        count = 1
        for extent in shape:
            count *= extent
        x, r, s_, o = (tensor(shape, DataType.BF16) for _ in range(4))
        w = tensor((1, cols), DataType.BF16)
        # four launches per event pair: the host's submission time hides behind the queue
        record(names[0], (2 * count + cols) * 2,
               lambda: ok(queue.rmsnorm(x.view(), w.view(), o.view(), eps)), str(list(shape)), inner=4)
        record(names[1], (4 * count + cols) * 2,
               lambda: ok(queue.add_rmsnorm(x.view(), r.view(), w.view(), s_.view(), o.view(), eps)),
               str(list(shape)), inner=4)
        record(names[2], (2 * count + cols) * 2,
               lambda: ok(queue.rmsnorm(x.view(), w.view(), o.view(), eps, order=1)),
               str(list(shape)), inner=4)
        release()
    if only is None or only in ("copy_bf16", "cast_bf16_f32", "cast_f32_bf16", "sumsq_bf16"):
        x, o = tensor((M, N), DataType.BF16), tensor((M, N), DataType.BF16)
        f = tensor((M, N), DataType.F32)
        record("copy_bf16", 2 * E * 2, lambda: ok(queue.copy(x.view(), o.view())), f"[{M},{N}]")
        record("cast_bf16_f32", 6 * E, lambda: ok(queue.cast(x.view(), f.view())), f"[{M},{N}]")
        record("cast_f32_bf16", 6 * E, lambda: ok(queue.cast(f.view(), o.view())), f"[{M},{N}]")
        scratch = device.create_workspace(int(lib.iomb_sumsq_scratch_bytes()))
        cell = device.create_workspace(32)

        def sumsq():
            return ok(queue.sumsq(x.view(), scratch.view(), cell.view().address()))
        record("sumsq_bf16", E * 2, sumsq, f"[{M},{N}]")
        scratch.close()
        cell.close()
        release()
    if only is None or only in ("silu_bf16", "silu_mul_bf16", "silu_then_mul_bf16", "silu_f32"):
        # Decoder MLP gate, TinyLlama geometry (intermediate 5632), 32768 rows: 369 MB per tensor.
        rows, inter = 32768, 5632
        count = rows * inter
        g, u, a, o = (tensor((rows, inter), DataType.BF16) for _ in range(4))
        record("silu_bf16", 2 * count * 2, lambda: ok(queue.silu(g.view(), a.view())),
               f"[{rows},{inter}]")
        record("silu_mul_bf16", 3 * count * 2,
               lambda: ok(queue.silu_mul(g.view(), u.view(), o.view())), f"[{rows},{inter}]")

        def silu_then_mul():
            ok(queue.silu(g.view(), a.view()))
            return ok(queue.mul(a.view(), u.view(), o.view()))
        # The unfused pair moves 5 tensors; its figure counts the fused op's 3 so that
        # the two lines compare the same useful work.
        record("silu_then_mul_bf16", 3 * count * 2, silu_then_mul, f"[{rows},{inter}] two launches")
        release()
        gf, af = tensor((rows // 2, inter), DataType.F32), tensor((rows // 2, inter), DataType.F32)
        record("silu_f32", 2 * (count // 2) * 4, lambda: ok(queue.silu(gf.view(), af.view())),
               f"[{rows // 2},{inter}]")
        release()
    if only is None or only in ("rope_bf16",):
        # Rotary embedding of Q at prefill, TinyLlama geometry: 32 heads x 64, 8192 positions,
        # 16 sequences: 537 MB per tensor; the 2 MiB angle table stays in L2.
        shape = (16, 32, 8192, 64)
        count = 16 * 32 * 8192 * 64
        q_in, q_out = tensor(shape, DataType.BF16), tensor(shape, DataType.BF16)
        record("rope_bf16", 2 * count * 2, lambda: ok(queue.rope(q_in.view(), q_out.view(), 0, 10000.0)),
               str(list(shape)))
        release()
    if only is None or only in ("sdpa_scale_mask", "sdpa_softmax", "sdpa_scale_mask_softmax",
                                "sdpa_canonicalize_output"):
        # Attention stages at TinyLlama prefill geometry: 32 heads, 2048 query rows against
        # 2048 cached tokens from an empty cache (a = 0): FP32 scores 537 MB, BF16
        # probabilities 268 MB. Algorithmic bytes: a visible score is read (and, for
        # scale/mask, written) once, every probability cell below L is written once.
        from iom_b200.device import SdpaStages
        heads, rows_q, tokens = 32, 2048, 2048
        ws = device.create_workspace(SdpaStages.workspace_bytes(1, heads, rows_q, tokens))
        stages = SdpaStages(ws.view(), 1, heads, 4, rows_q, tokens, 64, 0, tokens)
        ws.tensor()[:stages.cells * 4].view(torch.float32).copy_(
            torch.randn(stages.cells, device=device.torch_device) * 8.0)
        visible = heads * sum(min(tokens, r + 1) for r in range(rows_q))
        below = heads * rows_q * tokens
        note = f"Hq {heads}, R {rows_q}, L {tokens}, a 0"
        if only is None or only == "sdpa_softmax":
            record("sdpa_softmax", visible * 4 + below * 2, lambda: ok(queue.sdpa_softmax(stages)), note)
        if only is None or only == "sdpa_scale_mask_softmax":
            record("sdpa_scale_mask_softmax", visible * 4 + below * 2,
                   lambda: ok(queue.sdpa_scale_mask_softmax(stages)), note + ", scores only read")
        if only is None or only == "sdpa_scale_mask":
            # last: it rescales the scores in place on every launch
            record("sdpa_scale_mask", visible * 8, lambda: ok(queue.sdpa_scale_mask(stages)), note)
        ws.close()
        if only is None or only == "sdpa_canonicalize_output":
            merged = tensor((16, 8192, 2048), DataType.BF16)
            record("sdpa_canonicalize_output", 16 * 8192 * 2048 * 2,
                   lambda: ok(queue.sdpa_canonicalize_output(merged.view())),
                   "[16,8192,2048] read, nothing to rewrite")
            release()
    if only is None or only in ("embedding_prefill", "cache_append_prefill"):
        # Prefill-sized data movement: 131072 token rows of the TinyLlama table (537 MB out),
        # and 64 sequences x 4 KV heads x 2048 new rows appended into 4096-row caches.
        table = tensor((32000, 2048), DataType.BF16)
        count = 131072
        ids = device.create_tensor(TensorSpec((1, count), DataType.U32))
        made.append(ids)
        ids.storage().view(torch.int32).copy_(
            torch.randint(0, 32000, (ids.storage_nbytes // 4,), device=device.torch_device,
                          dtype=torch.int32))
        out = tensor((count, 2048), DataType.BF16)
        ws = device.create_workspace(32)
        record("embedding_prefill", 2 * count * 2048 * 2 + count * 4,
               lambda: ok(queue.embedding(table.view(), ids.view(), out.view(), ws.view())),
               f"table [32000,2048], {count} ids")
        ws.close()
        release()
        k = tensor((64, 4, 2048, 64), DataType.BF16)
        cache = tensor((64, 4, 4096, 64), DataType.BF16)
        record("cache_append_prefill", 2 * 64 * 4 * 2048 * 64 * 2,
               lambda: ok(queue.cache_append(k.view(), cache.view(), 1024)),
               "K [64,4,2048,64] -> cache [64,4,4096,64] at row 1024")
        release()
    if only is None or only in ("embedding_decode", "cache_append_decode_batched",
                                "cache_append_decode_64calls", "cast_logits"):
        # Decode-step data movement, TinyLlama geometry (the decode-step configuration): microseconds.
        table = tensor((32000, 2048), DataType.BF16)
        ids = device.create_tensor(TensorSpec((1, 64), DataType.U32))
        made.append(ids)
        ids.storage().view(torch.int32)[:64].copy_(
            torch.randint(0, 32000, (64,), device=device.torch_device, dtype=torch.int32))
        # ids of tile columns 1..3 start at slot 256, 512, 768 of the [1,64] plane
        raw = ids.storage().view(torch.int32)
        host_ids = torch.randint(0, 32000, (64,), dtype=torch.int32)
        for tile in range(4):
            raw[tile * 256:tile * 256 + 16].copy_(host_ids[tile * 16:(tile + 1) * 16])
        out = tensor((64, 2048), DataType.BF16)
        ws = device.create_workspace(32)
        record("embedding_decode", 2 * 64 * 2048 * 2 + 64 * 4 + 4,
               lambda: ok(queue.embedding(table.view(), ids.view(), out.view(), ws.view())),
               "table [32000,2048], 64 ids", inner=12)
        k = tensor((64, 4, 1, 64), DataType.BF16)
        cache = tensor((64, 4, 2048, 64), DataType.BF16)
        positions = torch.randint(0, 2047, (64,), device=device.torch_device, dtype=torch.int32)
        status = torch.zeros(8, device=device.torch_device, dtype=torch.int32)

        def batched():
            return ok(queue.cache_append_batched(k.view(), cache.view(), positions.data_ptr(),
                                                 status.data_ptr()))
        record("cache_append_decode_batched", 2 * 64 * 4 * 64 * 2, batched,
               "K [64,4,1,64] -> cache [64,4,2048,64], one call", inner=12)
        host_positions = positions.cpu().tolist()

        def per_sequence():
            for b in range(64):
                token = ok(queue.cache_append(k.view().select(0, b), cache.view().select(0, b),
                                              host_positions[b]))
            return token
        record("cache_append_decode_64calls", 2 * 64 * 4 * 64 * 2, per_sequence,
               "the contract form: 64 calls on select(0,b) views")
        logits = tensor((64, 32000), DataType.BF16)
        wide = tensor((64, 32000), DataType.F32)
        record("cast_logits", 64 * 32000 * 6, lambda: ok(queue.cast(logits.view(), wide.view())),
               "[64,32000] BF16 -> F32", inner=12)
        ws.close()
        release()
    if only is None or only in ("decode_step_eager", "decode_step_graph"):
        # One decode step's tensor-op traffic, TinyLlama geometry, 64 sequences, 22 layers:
        # embedding, then per layer norm / K,V appends / residual add + norm / gate / residual
        # add, then the final norm: 156 launches of microsecond-scale kernels. Eager: one
        # submission per launch through the host layer; graph: the whole step recorded once
        # (B200Queue.capture) and replayed as a single CUDA graph launch.
        batch, hidden, inter, layers, heads = 64, 2048, 5632, 22, 4
        table = tensor((32000, hidden), DataType.BF16)
        ids = device.create_tensor(TensorSpec((1, batch), DataType.U32))
        made.append(ids)
        ids.storage().zero_()
        h, normed, attn, total = (tensor((batch, hidden), DataType.BF16) for _ in range(4))
        w = tensor((1, hidden), DataType.BF16)
        gate, up, prod = (tensor((batch, inter), DataType.BF16) for _ in range(3))
        k, v = tensor((batch, heads, 1, 64), DataType.BF16), tensor((batch, heads, 1, 64), DataType.BF16)
        k_cache = tensor((batch, heads, 512, 64), DataType.BF16)
        v_cache = tensor((batch, heads, 512, 64), DataType.BF16)
        positions = torch.randint(0, 511, (batch,), device=device.torch_device, dtype=torch.int32)
        status = torch.zeros(8, device=device.torch_device, dtype=torch.int32)
        ws = device.create_workspace(32)

        def step():
            token = ok(queue.embedding(table.view(), ids.view(), h.view(), ws.view()))
            for _ in range(layers):
                queue.rmsnorm(h.view(), w.view(), normed.view(), 1e-5)
                queue.cache_append_batched(k.view(), k_cache.view(), positions.data_ptr(),
                                           status.data_ptr())
                queue.cache_append_batched(v.view(), v_cache.view(), positions.data_ptr(),
                                           status.data_ptr())
                queue.add_rmsnorm(h.view(), attn.view(), w.view(), total.view(), normed.view(), 1e-5)
                queue.silu_mul(gate.view(), up.view(), prod.view())
                token = queue.add(total.view(), attn.view(), h.view())
            if token != OID_CAPTURED:
                ok(token)
            return queue.rmsnorm(h.view(), w.view(), normed.view(), 1e-5)

        from iom_b200.device import OID_CAPTURED
        launches = 2 + layers * 6
        moved = (2 * batch * hidden * 2) + layers * (
            2 * batch * hidden * 2 + 2 * 2 * batch * heads * 64 * 2 + 4 * batch * hidden * 2
            + 3 * batch * inter * 2 + 3 * batch * hidden * 2) + 2 * batch * hidden * 2
        record("decode_step_eager", moved, lambda: ok(step()), f"{launches} launches, one submission each")
        if only is None or only == "decode_step_graph":
            queue.wait(ok(step()))
            with queue.capture() as recorded:
                step()
            record("decode_step_graph", moved, lambda: ok(recorded.replay()),
                   f"{launches} launches, one graph replay")
        ws.close()
        release()
    return results


def elementwise_sweep(device, queue, iters: int = 5) -> dict:
    """The mixed elementwise sweep: I32 ADD, F32 MUL and BF16 ADD with full-shape, row-broadcast
    [1,N] and column-broadcast [M,1] operands over 2^16 .. 2^30 elements, doubling
    (shape [E / 2048, 2048]). Device-resident GB/s of algorithmic bytes per size;
    sizes below the 126 MB L2 run out of cache and are reported as they are."""
    import torch

    from iom_b200.tensor import DataType, TensorSpec

    n = 2048
    results = {}
    for dtype, name, b, op in ((DataType.I32, "add_i32", 4, "add"), (DataType.F32, "mul_f32", 4, "mul"),
                               (DataType.BF16, "add_bf16", 2, "add")):
        for exponent in range(16, 31):
            elements = 1 << exponent
            m = elements // n
            tensors = [device.create_tensor(TensorSpec(shape, dtype))
                       for shape in ((m, n), (m, n), (m, n), (1, n), (m, 1))]
            for t in tensors:
                t.storage().copy_(torch.randint(0, 64, (t.storage_nbytes,), device=device.torch_device,
                                                dtype=torch.uint8))
            x, y, o, row, col = tensors
            fn = getattr(queue, op)
            torch.cuda.synchronize()    # the fills above run on another stream
            for form, rhs, nbytes in (("full", y, 3 * elements * b), ("row", row, (2 * elements + n) * b),
                                      ("col", col, (2 * elements + m) * b)):
                for _ in range(2):
                    token = fn(x.view(), rhs.view(), o.view())
                queue.wait(token)
                pairs = []
                for _ in range(iters):
                    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a0.record(queue.stream)
                    token = fn(x.view(), rhs.view(), o.view())
                    a1.record(queue.stream)
                    pairs.append((a0, a1))
                queue.wait(token)
                torch.cuda.synchronize()
                ms = sorted(p[0].elapsed_time(p[1]) for p in pairs)[len(pairs) // 2]
                results[f"{name}_{form}_2^{exponent}"] = {"GB/s": nbytes / ms / 1e6, "us": ms * 1e3}
            for t in tensors:
                t.close()
    return results


# ---- CPU side: the reference's own CPU backend (or the oracle port) ---------------

def _cpu_arm(threads: int, repeats: int, warmup: int) -> dict:
    """Times add(x, r, s) followed by rmsnorm(s, w, n) — the reference's contract
    path for this step — on `threads` independent row shards, one reference
    device + queue (one worker thread) per shard. Bytes are counted like the GPU
    arm's (fused-equivalent algorithmic bytes for the rows processed) so the two
    GB/s figures describe the same amount of work."""
    import ctypes

    import numpy as np
    import support
    from iom_b200.tensor import DataType

    kind = None
    for candidate in ("avx512", "portable"):
        if support.REF_LIBS[candidate].exists():
            probe = support.Reference(candidate)
            active = probe.lib.iomref_avx512_bf16_active() == 1
            probe.close()
            if candidate == "portable" or active:
                kind = candidate
                break
    rng = np.random.default_rng(7)

    def payloads(rows):
        x = support.f32_to_bf16_bits(rng.standard_normal((rows, HIDDEN), dtype=np.float32))
        r = support.f32_to_bf16_bits(rng.standard_normal((rows, HIDDEN), dtype=np.float32))
        w = support.f32_to_bf16_bits(
            (1.0 + 0.02 * rng.standard_normal((1, HIDDEN))).astype(np.float32))
        return x, r, w

    if kind is None:
        # Oracle port: scalar plain-C restatement, one core.
        rows, threads = 128, 1
        x, r, w = payloads(rows)
        hosts = {}
        for name, data in (("x", x), ("r", r), ("w", w), ("s", x), ("n", x)):
            tensor = support.HostTensor(data.shape, DataType.BF16)
            tensor.view().copy_from_host(data)
            hosts[name] = tensor
        lib = support.oracle()

        def once():
            assert lib.iomo_binary(0, support.abi(hosts["x"].view()), support.abi(hosts["r"].view()),
                                   support.abi(hosts["s"].view()), 0) == 0
            assert lib.iomo_rmsnorm(support.abi(hosts["s"].view()), support.abi(hosts["w"].view()),
                                    support.abi(hosts["n"].view()), EPS, 1) == 0
        label, sample_kind = "oracle port (plain C, scalar codec)", "port"
    else:
        rows = 4096 if kind == "avx512" else 128
        shards = []
        for _ in range(threads):
            ref = support.Reference(kind)
            x, r, w = payloads(rows)
            tensors = {}
            for name, data in (("x", x), ("r", r), ("w", w), ("s", x), ("n", x)):
                tensor = ref.tensor(data.shape, DataType.BF16)
                tensor.view().from_host(data)
                tensors[name] = tensor.view()
            shards.append((ref, tensors))

        def once():
            tokens = []
            for ref, t in shards:
                a = ref.lib.iomref_binary(ref.queue, 0, t["x"].handle, t["r"].handle, t["s"].handle)
                b = ref.lib.iomref_rmsnorm(ref.queue, t["s"].handle, t["w"].handle, t["n"].handle,
                                           ctypes.c_float(EPS))
                assert a > 0 and b > 0, ref.error()
                tokens.append((ref, b))
            for ref, token in tokens:
                assert ref.lib.iomref_wait(ref.queue, token) == 0, ref.error()
        label = f"reference CPU backend, {kind} build (oracle/_ref)"
        sample_kind = "reference"

    for _ in range(warmup):
        once()
    samples = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        once()
        samples.append(time.perf_counter() - t0)
    seconds = statistics.median(samples)
    elements = threads * rows * HIDDEN
    bytes_per_step = 4 * elements * ELEM + threads * HIDDEN * ELEM
    return {"value": bytes_per_step / seconds / 1e9, "unit": "GB/s", "cores": threads,
            "kind": sample_kind,
            "sample": f"{label}: add + rmsnorm on {threads} shard(s) of [{rows},{HIDDEN}] BF16, "
                      f"median of {repeats} runs, {seconds * 1e3:.1f} ms per run",
            "ms_per_step": seconds * 1e3}


def run_reference(args) -> dict | None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    world = int(os.environ.get("WORLD_SIZE", "1"))
    threads = max(1, min(os.cpu_count() or 1, 64))
    cpu = _cpu_arm(threads, repeats=max(1, args.steps), warmup=max(1, min(args.warmup, 2)))
    return {
        "impl": "reference",
        "metric": METRIC,
        "value": cpu["value"],
        "unit": "GB/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": cpu["ms_per_step"],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32 accumulate, bf16 storage",
        "data": "synthetic (seeded normal, the TinyLlama prefill configuration's distributions)",
        "config": {"workload": WORKLOAD, "sample": cpu["sample"]},
        "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cpu["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-ops", action="store_true",
                        help="skip the per-operation table (N=1 only)")
    parser.add_argument("--op", default=None,
                        help="run one row of the per-operation table and print it "
                             "(for profiler captures), e.g. --op rmsnorm_c5shard")
    parser.add_argument("--sweep", action="store_true",
                        help="run the elementwise size sweep and print its table")
    parser.add_argument("--no-e2e", action="store_true",
                        help="skip the host-buffer leg (used for profiler captures)")
    parser.add_argument("--planes", type=int, default=PLANES,
                        help="planes of [8192,2048] per step; smaller values give the "
                             "small case profiler captures use")
    args = parser.parse_args()
    configure(args.planes)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.sweep:
        from iom_b200.device import DeviceMemoryConfig, make_b200_device
        device = make_b200_device(0, DeviceMemoryConfig(14 << 30))
        queue = device.create_ops()
        print(json.dumps({"sweep": "mixed elementwise sweep, [E/2048, 2048], E = 2^16 .. 2^30",
                          "result": elementwise_sweep(device, queue, iters=max(1, min(args.steps, 7)))}))
        queue.close()
        return
    if args.op is not None:
        import torch

        from iom_b200.device import DeviceMemoryConfig, make_b200_device
        torch.cuda.set_device(0)
        device = make_b200_device(0, DeviceMemoryConfig(5 << 30))
        queue = device.create_ops()
        print(json.dumps({"op": args.op, "result": ops_table(device, queue, only=args.op,
                                                             iters=max(1, args.steps))}))
        queue.close()
        return
    if args.impl == "reference":
        result = run_reference(args)
    else:
        result = run_ours(args)
        if result is not None and result["n_gpus"] == 1 and not args.no_cpu_baseline:
            cpu = _cpu_arm(1, repeats=3, warmup=1)
            result["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    restore = getattr(args, "_restore_stdout", None)
    if restore is not None:
        sys.stdout.flush()
        restore()
    if result is not None:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
