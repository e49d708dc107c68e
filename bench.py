#!/usr/bin/env python
"""Benchmark of the hot path: residual ADD fused into RMSNorm on tiled BF16 storage.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

The workload is the large sharded configuration: BF16 [262144, 8192] residual ADD +
RMSNorm (eps 1e-6, x, r ~ N(0,1), scale ~ N(1, 0.02)), 17.2 GB of algorithmic traffic per
step. With N GPUs (one process per GPU, torchrun) the rows are cut on 16-row band
boundaries (iom_b200.sharding.shard_rows): rank k owns rows/N rows in its own GPU's
memory, the scale row is replicated, and no data-path collective exists ("scaling":
"strong"). A step is one iomb_add_rmsnorm launch over the rank's shard, issued through
the C++ backend (libiom_b200_backend.so, b200::add_rmsnorm on a device from
make_b200_device) and timed with CUDA events on the queue's stream, max over ranks. The
one exchange of the path, the whole-tensor FP32 sum of squares, is timed separately:
per-rank iomb_sumsq, NCCL all_gather of one float per rank, rank-ordered FP32 addition.

`e2e` is the same step through the reference's public interface with host buffers:
TensorView::copy_from_host(x), copy_from_host(residual), add_rmsnorm, wait,
copy_to_host(out), pinned host memory in the logical row-major layout, every step.

`--impl reference` times the reference's own CPU backend (oracle/_ref when the shim is
built, else the plain-C oracle port) on the host cores, on bounded row shards of the same
workload.
"""
from __future__ import annotations

import argparse
import json
import os
import re
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

ROWS, HIDDEN, EPS = 262144, 8192, 1e-6
ELEM = 2
METRIC = "achieved HBM GB/s, fused residual ADD + RMSNorm (BF16 [262144,8192], row-sharded)"
# dram__bytes_read.sum and dram__bytes_write.sum of one launch of the kernel the step runs,
# from the ncu capture summarised in profiles/add_rmsnorm_bf16_long_rows.md (a [32768,8192]
# shard in one launch: 2.15 GB, 17 times the L2). Reads are proportional to the rows. Writes
# are the algorithmic bytes less the lines still dirty in L2 when the launch ends, which
# does not grow with the rows.
NCU_READ_BYTES_PER_ROW = 1075119000 / 32768      # dram__bytes_read.sum of the 32768-row launch
NCU_WRITES_LEFT_IN_L2_BYTES = 32768 * 2 * 8192 * 2 - 1026173000   # algorithmic - dram__bytes_write.sum


def configure(rows: int) -> None:
    """Resizes the tensor (the default is the benchmark's; profiler captures shrink it)."""
    global ROWS
    ROWS = rows


def workload(world: int) -> str:
    per_rank = f"{ROWS // world} rows per rank on {world} rank(s)" if world > 1 else "one GPU holds all rows"
    return (f"C5: BF16 [{ROWS},{HIDDEN}] residual ADD + RMSNorm, eps 1e-6, x,r ~ N(0,1) seed 2, "
            f"w ~ N(1,0.02), row-sharded on band boundaries; {per_rank}")


def step_bytes(rows: int) -> int:
    """x and residual read, rounded sum and normalised output written, scale read once."""
    return 4 * rows * HIDDEN * ELEM + HIDDEN * ELEM


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
        self.lines = []          # (arrival time, text)
        self.begin = self.end = None

    def mark_begin(self):
        """The timed region starts here (the sampler itself was started earlier, so that
        nvidia-smi is already reporting)."""
        self.begin = time.monotonic()

    def mark_end(self):
        self.end = time.monotonic()

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            deadline = time.monotonic() + 2.0      # until nvidia-smi reports
            while not self.lines and time.monotonic() < deadline:
                time.sleep(0.01)
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

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
        for arrival, line in self.lines:
            # A sample describes the interval before its arrival.
            if self.begin is not None and arrival < self.begin + 0.01:
                continue
            if self.end is not None and arrival > self.end + 0.03:
                continue
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


def fill_normal_bf16(storage, seed: int, mean: float = 0.0, deviation: float = 1.0) -> None:
    """Fills a tiled BF16 owner (uint8 torch view of its storage) with seeded normal values,
    a gigabyte at a time. The tiled layout of independent samples is independent samples, so
    the values go straight into storage."""
    import torch

    generator = torch.Generator(device=storage.device)
    generator.manual_seed(seed)
    words = storage.view(torch.bfloat16)
    chunk = 1 << 27
    for start in range(0, words.numel(), chunk):
        part = words[start:start + chunk]
        part.copy_(torch.randn(part.numel(), device=storage.device, generator=generator,
                               dtype=torch.float32).mul_(deviation).add_(mean))


def run_ours(args) -> dict:
    import numpy as np
    import torch
    import torch.distributed as dist

    from iom_b200 import _abi, backend_driver as bd
    from iom_b200.sharding import all_gather_sum, shard_rows
    from iom_b200.tensor import DataType

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

    first_row, rows = shard_rows(ROWS, world, rank)
    elements = rows * HIDDEN
    tensor_bytes = elements * ELEM
    kernel_lib = _abi.load_library()
    # Arena: the shard's four tensors, the host-transfer staging range, small change.
    arena = 4 * tensor_bytes + (0 if args.no_e2e else 3 * tensor_bytes + (1 << 20)) + (256 << 20)
    backend = bd.Backend(local_rank, arena)
    x, r, total, out = (backend.tensor((rows, HIDDEN), DataType.BF16) for _ in range(4))
    scale = backend.tensor((1, HIDDEN), DataType.BF16)
    vx, vr, vt, vo, vw = (backend.view(t) for t in (x, r, total, out, scale))
    # Seeded inputs, generated on the device (seed 2, one stream per rank and operand).
    fill_normal_bf16(backend.storage(x), seed=2 + 1000 * rank)
    fill_normal_bf16(backend.storage(r), seed=2 + 1000 * rank + 500)
    rng = np.random.default_rng(2)
    w_host = (1.0 + 0.02 * rng.standard_normal((1, HIDDEN))).astype(np.float32)
    w_bits = ((w_host.view(np.uint32).astype(np.uint64) + 0x7FFF
               + ((w_host.view(np.uint32) >> 16) & 1)) >> 16).astype(np.uint16)
    small = backend.workspace(1 << 20)
    backend.run([bd.Backend.op(bd.FROM_HOST, [vw], workspace=small, host=w_bits.ctypes.data,
                               host_bytes=w_bits.nbytes)])
    torch.cuda.synchronize()

    step = [bd.Backend.op(bd.ADD_RMSNORM, [vx, vr, vw, vt, vo], eps=EPS)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput (`value`) -----------------------------
    with ClockSampler(local_rank) as sampler:
        backend.run(step, passes=args.warmup)
        kernel_name = (kernel_lib.iomb_last_launch() or b"").decode()
        barrier()
        sampler.mark_begin()
        timing = backend.run(step, passes=args.steps)
        barrier()
        sampler.mark_end()
    elapsed_ms = float(timing.device_ms)
    clocks = sampler.summary()

    # ---- end to end through the public interface with host buffers (`e2e`) -------
    e2e_ms = float("nan")
    e2e_sync_ms = float("nan")
    e2e_submit_us = None
    if not args.no_e2e:
        pinned = {name: torch.empty(tensor_bytes, dtype=torch.uint8, pin_memory=True)
                  for name in ("x", "r", "out")}
        # Host copies of the inputs in the logical row-major layout (any seeded values do:
        # the timing does not depend on them, the device-resident leg's values are used).
        pinned["x"].copy_(backend.storage(x))
        pinned["r"].copy_(backend.storage(r))
        staging = backend.workspace(tensor_bytes + 64)
        staging_down = backend.workspace(tensor_bytes + 64)
        out_b = backend.tensor((rows, HIDDEN), DataType.BF16)
        outs = [vo, backend.view(out_b)]

        def upload_and_compute(destination):
            return [
                bd.Backend.op(bd.FROM_HOST, [vx], workspace=staging, host=pinned["x"].data_ptr(),
                              host_bytes=tensor_bytes),
                bd.Backend.op(bd.FROM_HOST, [vr], workspace=staging, host=pinned["r"].data_ptr(),
                              host_bytes=tensor_bytes),
                bd.Backend.op(bd.ADD_RMSNORM, [vx, vr, vw, vt, destination], eps=EPS),
                bd.Backend.op(bd.WAIT),
            ]

        def download(source):
            return [bd.Backend.op(bd.TO_HOST, [source], workspace=staging_down,
                                  host=pinned["out"].data_ptr(), host_bytes=tensor_bytes)]

        # (a) One host thread, the contract's synchronous calls one after another.
        synchronous = upload_and_compute(vo) + download(vo)
        backend.run(synchronous, passes=1)
        barrier()
        sync_steps = min(args.steps, 8)
        sync_timing = backend.run(synchronous, passes=sync_steps)
        barrier()
        e2e_sync_ms = sync_timing.host_seconds * 1e3 / sync_steps

        # (b) The same synchronous calls from two host threads: one uploads and computes
        # step s + 1 while the other reads the result of step s back (two output tensors
        # in turn), so both directions of the host link are busy. Every step still moves
        # its inputs in and its result out inside the timed region.
        failures = []
        computed = [threading.Semaphore(0), threading.Semaphore(0)]
        drained = [threading.Semaphore(1), threading.Semaphore(1)]

        def producer(count):
            try:
                for s_index in range(count):
                    drained[s_index % 2].acquire()
                    backend.run(upload_and_compute(outs[s_index % 2]), passes=1)
                    computed[s_index % 2].release()
            except Exception as error:          # noqa: BLE001 - reported by the main thread
                failures.append(error)
                for semaphore in computed:
                    semaphore.release()

        def consumer(count):
            try:
                for s_index in range(count):
                    computed[s_index % 2].acquire()
                    if failures:
                        return
                    backend.run(download(outs[s_index % 2]), passes=1)
                    drained[s_index % 2].release()
            except Exception as error:          # noqa: BLE001
                failures.append(error)
                for semaphore in drained:
                    semaphore.release()

        def pipelined(count):
            threads = [threading.Thread(target=producer, args=(count,)),
                       threading.Thread(target=consumer, args=(count,))]
            begin = time.perf_counter()
            for thread in threads:
                thread.start()
            for thread in threads:
                thread.join()
            if failures:
                raise failures[0]
            return (time.perf_counter() - begin) * 1e3

        pipelined(2)
        barrier()
        e2e_ms = pipelined(args.steps)
        barrier()

    # ---- whole-tensor sum of squares across ranks (the one exchange step) ----
    sumsq_bytes = 32 + int(kernel_lib.iomb_sumsq_scratch_bytes())
    sumsq_workspace = backend.workspace(sumsq_bytes)
    # the workspace is leased for each call: wait before the next one names it again
    sumsq_program = [bd.Backend.op(bd.SUMSQ, [vt], workspace=sumsq_workspace), bd.Backend.op(bd.WAIT)]
    backend.run(sumsq_program, passes=2)
    barrier()
    sumsq_timing = backend.run(sumsq_program, passes=5)
    local = backend.workspace_memory(sumsq_workspace, 4).view(torch.float32)
    sumsq_info = {"kernel_ms_per_rank": float(sumsq_timing.device_ms) / 5,
                  "bytes_read_per_rank": tensor_bytes,
                  "kernel_GB/s_per_rank": tensor_bytes / (float(sumsq_timing.device_ms) / 5) / 1e6}
    if world > 1:
        combined = all_gather_sum(local.clone())
        barrier()
        t0 = time.perf_counter()
        for _ in range(5):
            backend.run(sumsq_program, passes=1)
            combined = all_gather_sum(local.clone())
        torch.cuda.synchronize()
        sumsq_info["ms_with_combine"] = (time.perf_counter() - t0) * 1e3 / 5
        gathered = [torch.empty_like(combined.reshape(1)) for _ in range(world)]
        dist.all_gather(gathered, combined.reshape(1))
        sumsq_info.update({
            "value": float(combined),
            "identical_on_all_ranks": all(torch.equal(gathered[0], g) for g in gathered),
            "combine": "all_gather of one FP32 partial per rank, added in rank order"})
    else:
        sumsq_info["value"] = float(local.cpu()[0])

    backend.close()
    table = None
    if world == 1 and not args.no_ops:
        table = ops_table_all(local_rank)

    times = torch.tensor([elapsed_ms, e2e_ms, e2e_sync_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, e2e_sync_ms = (float(v) for v in times.tolist())

    result = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        per_launch_ms = elapsed_ms / args.steps
        total_bytes = step_bytes(ROWS) + (world - 1) * HIDDEN * ELEM
        achieved = step_bytes(rows) / per_launch_ms / 1e6        # this rank's kernel
        # DRAM traffic of one step from the ncu capture of a [32768,8192] shard: reads scale
        # with the rows; so do writes, except for the lines still dirty in L2 when the last
        # launch ends (bounded by the L2 size, the same at every row count), which the DRAM
        # counters of a kernel never see.
        traffic = None
        if NCU_READ_BYTES_PER_ROW is not None:
            traffic = (NCU_READ_BYTES_PER_ROW * rows + 2 * HIDDEN * ELEM * rows
                       - NCU_WRITES_LEFT_IN_L2_BYTES)
        found = re.search(r"(\d+) launch\(es\)", kernel_name)
        launches_per_step = int(found.group(1)) if found else 1
        result = {
            "metric": METRIC,
            "value": total_bytes * args.steps / elapsed_ms / 1e6,
            "unit": "GB/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": per_launch_ms,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "f32 accumulate, bf16 storage",
            "data": "synthetic (seeded normal, the large sharded configuration's distributions)",
            "config": {"workload": workload(world), "launches_per_step": launches_per_step,
                       "rows_per_rank": rows, "first_row_of_rank_0": first_row,
                       "algorithmic_bytes_per_step": total_bytes,
                       "l2": f"inputs larger than L2 ({step_bytes(rows) / 1e9:.2f} GB touched per rank "
                             "and step, L2 is 126 MB)",
                       "order": "LANES16 (the reference's AVX-512 BF16 order)",
                       "host_layer": "C++ backend (libiom_b200_backend.so: b200::add_rmsnorm on a device "
                                     "from make_b200_device), launches issued from C++",
                       "timing": f"{args.steps} steps back to back between one pair of CUDA events "
                                 "on the queue's stream, max over ranks",
                       "pct_of_8TBps_per_gpu": 100.0 * achieved / 8000.0},
            "clocks": clocks,
            "e2e": {"value": total_bytes * args.steps / e2e_ms / 1e6 if e2e_ms == e2e_ms else None,
                    "unit": "GB/s",
                    "h2d_bytes_per_step": 2 * ROWS * HIDDEN * ELEM,
                    "d2h_bytes_per_step": ROWS * HIDDEN * ELEM,
                    "steps": args.steps,
                    "synchronous_value": (total_bytes / e2e_sync_ms / 1e6
                                          if e2e_sync_ms == e2e_sync_ms else None),
                    "path": "C++ backend through the reference's public interface, every step: "
                            "TensorView::copy_from_host(x), copy_from_host(residual), "
                            "b200::add_rmsnorm, wait, copy_to_host(out); pinned host buffers in the "
                            "logical row-major layout; host wall clock over all steps, max over ranks. "
                            "`value`: those synchronous calls from two host threads (one uploads and "
                            "computes step s+1 while the other reads step s back, two output tensors in "
                            "turn); `synchronous_value`: one thread, one call after another"},
            "gpu_launches": args.steps * launches_per_step,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one "
                                           "launch on a [32768,8192] shard, scaled by rows; writes "
                                           "still dirty in L2 at the end of the step are not DRAM "
                                           "traffic of the kernel (profiles/add_rmsnorm_bf16_long_rows.md)",
                         "launches": f"{launches_per_step} launch(es) of this kernel per step; achieved = "
                                     "algorithmic bytes of a step / duration of a step",
                         "peak_source": f"of {peak_kind}", "kernel": kernel_name,
                         "algorithmic_bytes_per_step": step_bytes(rows), "per": "GPU (rank 0's shard)"},
            "sumsq_across_ranks": sumsq_info,
        }
        if table is not None:
            result["ops"] = table
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result


def ops_table_all(ordinal: int) -> dict:
    """Per-operation supporting numbers: kernel-level GB/s through the Python mirror (several
    launches per event pair, so that its submission time hides behind the queue), and
    launch-bound sequences through the C++ backend."""
    from iom_b200.device import DeviceMemoryConfig, make_b200_device

    device = make_b200_device(ordinal, DeviceMemoryConfig(5 << 30))
    queue = device.create_ops()
    table = ops_table(device, queue)
    queue.close()
    del queue, device
    try:
        table.update(backend_sequences(ordinal))
    except Exception as error:      # the table is supporting material: report, do not fail the line
        table["cpp_backend_sequences"] = {"error": str(error)}
    return table


def backend_sequences(ordinal: int) -> dict:
    """Launch-bound work issued from C++ through the reference's facade on the B200 backend:
    the small sizes of the elementwise sweep (device time per launch and host time per
    submission), and one decode step's tensor operations (TinyLlama geometry, 64 sequences,
    22 layers) issued one by one and replayed from a recording."""
    import torch

    from iom_b200 import backend_driver as bd
    from iom_b200.tensor import DataType

    results = {}
    backend = bd.Backend(ordinal, 2 << 30)
    n = 2048
    for exponent in range(16, 23):
        m = (1 << exponent) // n
        a, b, o = (backend.tensor((m, n), DataType.F32) for _ in range(3))
        views = [backend.view(t) for t in (a, b, o)]
        timing = backend.run([bd.Backend.op(bd.MUL, views)], passes=200, warmup=20)
        nbytes = 3 * (1 << exponent) * 4
        results[f"mul_f32_full_2^{exponent}_cpp"] = {
            "us": timing.device_ms * 1e3 / 200, "GB/s": nbytes / (timing.device_ms / 200) / 1e6,
            "host_us_per_submission": timing.submit_seconds * 1e6 / 200,
            "note": "200 launches back to back from C++; sizes below the 126 MB L2 run out of cache"}
    batch, hidden, inter, layers, heads = 64, 2048, 5632, 22, 4
    table = backend.tensor((32000, hidden), DataType.BF16)
    ids = backend.tensor((1, batch), DataType.U32)
    backend.storage(ids).zero_()
    h, normed, attn, total = (backend.tensor((batch, hidden), DataType.BF16) for _ in range(4))
    w = backend.tensor((1, hidden), DataType.BF16)
    gate, up, prod = (backend.tensor((batch, inter), DataType.BF16) for _ in range(3))
    k, v = (backend.tensor((batch, heads, 1, 64), DataType.BF16) for _ in range(2))
    k_cache, v_cache = (backend.tensor((batch, heads, 512, 64), DataType.BF16) for _ in range(2))
    for t in (table, h, attn, w, gate, up, k, v):
        storage = backend.storage(t)
        storage.view(torch.bfloat16).copy_(torch.randn(storage.numel() // 2, device=storage.device))
    status_ws = backend.workspace(32)
    control = backend.workspace(32 + 4 * batch)
    backend.workspace_memory(control, 32 + 4 * batch).view(torch.int32)[8:].copy_(
        torch.randint(0, 511, (batch,), dtype=torch.int32))
    V = {name: backend.view(t) for name, t in (
        ("table", table), ("ids", ids), ("h", h), ("normed", normed), ("attn", attn), ("total", total),
        ("w", w), ("gate", gate), ("up", up), ("prod", prod), ("k", k), ("v", v),
        ("k_cache", k_cache), ("v_cache", v_cache))}
    op = bd.Backend.op
    program = [op(bd.EMBEDDING, [V["table"], V["ids"], V["h"]], workspace=status_ws)]
    for _ in range(layers):
        program += [
            op(bd.RMSNORM, [V["h"], V["w"], V["normed"]], eps=1e-5),
            op(bd.CACHE_APPEND_BATCHED, [V["k"], V["k_cache"]], workspace=control),
            op(bd.CACHE_APPEND_BATCHED, [V["v"], V["v_cache"]], workspace=control),
            op(bd.ADD_RMSNORM, [V["h"], V["attn"], V["w"], V["total"], V["normed"]], eps=1e-5),
            op(bd.SILU_MUL, [V["gate"], V["up"], V["prod"]]),
            op(bd.ADD, [V["total"], V["attn"], V["h"]]),
        ]
    program.append(op(bd.RMSNORM, [V["h"], V["w"], V["normed"]], eps=1e-5))
    # A decode step ends with the host reading the result: the step's tokens are collected
    # (which also returns the embedding's status-word lease before the next step).
    program.append(op(bd.WAIT))
    # The decode step's single operations and the other launches that last a few
    # microseconds, issued back to back from C++ (the per-operation table times them through
    # the Python mirror, whose submission costs more than these kernels run).
    logits = backend.tensor((batch, 32000), DataType.BF16)
    wide = backend.tensor((batch, 32000), DataType.F32)
    a_c1, o_c1 = (backend.tensor((4096, 2048), DataType.F32) for _ in range(2))
    bias_c1 = backend.tensor((1, 2048), DataType.F32)
    k_big = backend.tensor((batch, heads, 2048, 64), DataType.BF16)
    cache_big = backend.tensor((batch, heads, 4096, 64), DataType.BF16)
    singles = [
        ("embedding_decode_cpp", [op(bd.EMBEDDING, [V["table"], V["ids"], V["h"]], workspace=status_ws),
                                  op(bd.WAIT)],
         2 * batch * hidden * 2 + batch * 4 + 4, "table [32000,2048], 64 ids; waited for each time (the "
                                                 "status word is a lease)"),
        ("cache_append_decode_batched_cpp",
         [op(bd.CACHE_APPEND_BATCHED, [V["k"], V["k_cache"]], workspace=control)],
         2 * batch * heads * 64 * 2, "K [64,4,1,64] -> cache [64,4,512,64], one call"),
        ("cast_logits_cpp", [op(bd.CAST, [backend.view(logits), backend.view(wide)])],
         batch * 32000 * 6, "[64,32000] BF16 -> F32"),
        ("add_f32_row_config1_cpp",
         [op(bd.ADD, [backend.view(a_c1), backend.view(bias_c1), backend.view(o_c1)])],
         2 * 4096 * 2048 * 4 + 2048 * 4, "[4096,2048] + [1,2048], one buffer set (L2-resident)"),
        ("cache_append_prefill_cpp",
         [op(bd.CACHE_APPEND, [backend.view(k_big), backend.view(cache_big)], a=1024)],
         2 * batch * heads * 2048 * 64 * 2, "K [64,4,2048,64] -> cache [64,4,4096,64] at row 1024"),
        ("rmsnorm_decode_cpp", [op(bd.RMSNORM, [V["h"], V["w"], V["normed"]], eps=1e-5)],
         2 * batch * hidden * 2, "[64,2048] BF16"),
    ]
    for name, single, nbytes, note in singles:
        timing = backend.run(single, passes=200, warmup=20)
        results[name] = {
            "us": timing.device_ms * 1e3 / 200, "GB/s": nbytes / (timing.device_ms / 200) / 1e6,
            "host_us_per_submission": timing.submit_seconds * 1e6 / 200,
            "note": note + "; 200 launches back to back from C++, CUDA events around them"}
    launches = sum(1 for record in program if record.opcode != bd.WAIT)
    for name, mode in (("decode_step_eager_cpp", bd.EAGER), ("decode_step_recorded_cpp", bd.RECORDED)):
        plain = [record for record in program if record.opcode != bd.WAIT] if mode == bd.RECORDED else program
        timing = backend.run(plain, passes=50, warmup=5, mode=mode)
        results[name] = {
            "us": timing.device_ms * 1e3 / 50,
            "host_us_per_step": timing.host_seconds * 1e6 / 50,
            "host_us_per_submission": timing.submit_seconds * 1e6 / max(1, timing.operations),
            "launches": launches,
            "note": f"{launches} facade operations per step issued from C++"
                    + (", recorded once and replayed as one submission" if mode == bd.RECORDED else "")}
    backend.close()
    return results


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

    peak, peak_kind = measured_peak()

    def record(name, nbytes, launch, shape, inner=1):
        if only is not None and name != only:
            return
        ms = timed(launch, inner)
        results[name] = {"GB/s": nbytes / ms / 1e6, "us": ms * 1e3, "bytes": nbytes,
                         "pct_of_8TBps": nbytes / ms / 1e6 / 80.0,
                         f"frac_of_{peak_kind}_peak": nbytes / ms / 1e6 / peak, "shape": shape,
                         "timing": "one launch per CUDA-event pair, median" if inner == 1 else
                                   f"{inner} launches back to back per CUDA-event pair, median per launch"}

    if only is None or only == "add_f32_row_config1":
        # Configuration 1 as stated: F32 A[4096,2048] + bias[2048] -> C. One set is 64 MiB,
        # half the L2, so eight sets of (A, C) rotate: every launch streams from HBM.
        bias = tensor((1, 2048), DataType.F32)
        sets = [(tensor((4096, 2048), DataType.F32), tensor((4096, 2048), DataType.F32))
                for _ in range(8)]
        turn = [0]

        def config1():
            a_, c_ = sets[turn[0] % len(sets)]
            turn[0] += 1
            return ok(queue.add(a_.view(), bias.view(), c_.view()))
        record("add_f32_row_config1", (2 * 4096 * 2048 + 2048) * 4, config1,
               "[4096,2048] + [1,2048], eight rotating buffer sets", inner=8)
        release()
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
    for label, shape, eps in (("tinyllama", (16, 8192, 2048), 1e-5), ("c5shard", (32768, 8192), 1e-6),
                              # other row lengths of the long-row kernel (rows chaining at once
                              # on an SM shrink as the rows grow)
                              ("f4096", (65536, 4096), 1e-6), ("f16384", (16384, 16384), 1e-6)):
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
        if label in ("tinyllama", "c5shard"):
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
    if only is None or only in ("embedding_prefill", "embedding_prefill_sorted",
                                "embedding_prefill_repeated", "cache_append_prefill"):
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
        gather = lambda: ok(queue.embedding(table.view(), ids.view(), out.view(), ws.view()))  # noqa: E731
        if only in (None, "embedding_prefill"):
            record("embedding_prefill", 2 * count * 2048 * 2 + count * 4, gather,
                   f"table [32000,2048], {count} uniform random ids")
        # The same gather with ids in ascending order (neighbouring output rows read
        # neighbouring table rows), and with every id equal (one table row, always in cache):
        # what the table side of the random case costs.
        if only in (None, "embedding_prefill_sorted"):
            flat = ids.storage().view(torch.int32)
            flat.copy_(torch.sort(flat).values)
            record("embedding_prefill_sorted", 2 * count * 2048 * 2 + count * 4, gather,
                   f"table [32000,2048], {count} ids in ascending order")
        if only in (None, "embedding_prefill_repeated"):
            ids.storage().view(torch.int32).fill_(12345)
            record("embedding_prefill_repeated", count * 2048 * 2 + 2048 * 2 + count * 4, gather,
                   f"table [32000,2048], {count} equal ids (bytes: the output, one table row)")
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

def _reference_kind():
    """'avx512' when that build of the reference shim exists and this host can run it,
    'portable' when only that one exists, None when no shim was built."""
    import support

    for candidate in ("avx512", "portable"):
        if support.REF_LIBS[candidate].exists():
            probe = support.Reference(candidate)
            active = probe.lib.iomref_avx512_bf16_active() == 1
            probe.close()
            if candidate == "portable" or active:
                return candidate
    return None


def _cpu_arm(threads: int, repeats: int, warmup: int, force_kind=None) -> dict:
    """Times add(x, r, s) followed by rmsnorm(s, w, n) — the reference's contract
    path for this step — on `threads` independent row shards of the benchmark's tensor
    ([rows, 8192] BF16 each), one reference device + queue (one worker thread) per shard.
    Bytes are counted like the GPU arm's (fused-equivalent algorithmic bytes for the rows
    processed) so the two GB/s figures describe the same amount of work."""
    import ctypes

    import numpy as np
    import support
    from iom_b200.tensor import DataType

    kind = force_kind or _reference_kind()
    rng = np.random.default_rng(2)

    def payloads(rows):
        x = support.f32_to_bf16_bits(rng.standard_normal((rows, HIDDEN), dtype=np.float32))
        r = support.f32_to_bf16_bits(rng.standard_normal((rows, HIDDEN), dtype=np.float32))
        w = support.f32_to_bf16_bits(
            (1.0 + 0.02 * rng.standard_normal((1, HIDDEN))).astype(np.float32))
        return x, r, w

    if kind is None:
        # Oracle port: scalar plain-C restatement, one core.
        rows, threads = 32, 1
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
        # The AVX-512 BF16 build runs ~1 GB/s per core: 1024 rows (67 MB touched) per shard
        # and step; the portable build's bit-serial codec needs a 32-row slice.
        rows = 1024 if kind == "avx512" else 32
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
    total_rows = threads * rows
    bytes_per_step = 4 * total_rows * HIDDEN * ELEM + threads * HIDDEN * ELEM
    return {"value": bytes_per_step / seconds / 1e9, "unit": "GB/s", "cores": threads,
            "kind": sample_kind,
            "sample": f"{label}: add then rmsnorm on {threads} row shard(s) of [{rows},{HIDDEN}] BF16 "
                      f"({total_rows} of the tensor's {ROWS} rows per step; rows are independent, so the "
                      f"rate extrapolates), median of {repeats} runs, {seconds * 1e3:.1f} ms per run",
            "rows_per_step": total_rows,
            "ms_per_step": seconds * 1e3}


def cpu_per_op(threads: int) -> dict:
    """The five named operations on the reference CPU backend: steady clock around
    operation + wait, one warm-up and five samples, median (the method of
    test/cpu/test_cpu_bench.cpp:63-83), on `threads` shards in parallel queues and on one."""
    import ctypes

    import numpy as np
    import support
    from iom_b200.tensor import DataType

    kind = _reference_kind()
    if kind is None:
        return {"unavailable": "the reference CPU backend shim is not built"}
    rows = 1024 if kind == "avx512" else 16
    rng = np.random.default_rng(3)
    results = {"build": kind, "rows_per_shard": rows}

    def measure(make_shard, nbytes_per_shard, name, count):
        shards = [make_shard() for _ in range(count)]

        def once():
            pending = [(ref, launch()) for ref, launch in shards]
            for ref, token in pending:
                assert token > 0, ref.error()
                assert ref.lib.iomref_wait(ref.queue, token) == 0, ref.error()
        once()
        samples = []
        for _ in range(5):
            t0 = time.perf_counter()
            once()
            samples.append(time.perf_counter() - t0)
        seconds = statistics.median(samples)
        results[f"{name}_{count}core"] = {"GB/s": count * nbytes_per_shard / seconds / 1e9,
                                          "ms": seconds * 1e3, "cores": count}
        for ref, _ in shards:
            ref.close()

    def bf16(shape):
        return support.f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32))

    def binary_shard(op, dtype, rhs_shape):
        def make():
            ref = support.Reference(kind)
            shape = (rows, 2048)
            if dtype == DataType.BF16:
                a, b = bf16(shape), bf16(rhs_shape)
            elif dtype == DataType.F32:
                a = rng.uniform(-1, 1, shape).astype(np.float32)
                b = rng.uniform(-1, 1, rhs_shape).astype(np.float32)
            else:
                a = rng.integers(-(1 << 20), 1 << 20, shape).astype(np.int32)
                b = rng.integers(-(1 << 20), 1 << 20, rhs_shape).astype(np.int32)
            ta, tb, to = ref.tensor(shape, dtype), ref.tensor(rhs_shape, dtype), ref.tensor(shape, dtype)
            ta.view().from_host(a)
            tb.view().from_host(b)
            va, vb, vo = ta.view(), tb.view(), to.view()
            return ref, lambda: ref.lib.iomref_binary(ref.queue, op, va.handle, vb.handle, vo.handle)
        return make

    elem = {DataType.BF16: 2, DataType.F32: 4, DataType.I32: 4}
    for count in sorted({1, threads}):
        measure(binary_shard(0, DataType.F32, (1, 2048)), (2 * rows * 2048 + 2048) * 4,
                "add_f32_row_broadcast", count)
        measure(binary_shard(1, DataType.F32, (rows, 2048)), 3 * rows * 2048 * 4, "mul_f32_full", count)
        measure(binary_shard(0, DataType.BF16, (rows, 2048)), 3 * rows * 2048 * 2, "add_bf16_full", count)
        measure(binary_shard(0, DataType.I32, (rows, 2048)), 3 * rows * 2048 * 4, "add_i32_full", count)

        def rmsnorm_shard():
            ref = support.Reference(kind)
            tx, tw, to = (ref.tensor((rows, HIDDEN), DataType.BF16), ref.tensor((1, HIDDEN), DataType.BF16),
                          ref.tensor((rows, HIDDEN), DataType.BF16))
            tx.view().from_host(bf16((rows, HIDDEN)))
            tw.view().from_host(bf16((1, HIDDEN)))
            vx, vw, vo = tx.view(), tw.view(), to.view()
            return ref, lambda: ref.lib.iomref_rmsnorm(ref.queue, vx.handle, vw.handle, vo.handle,
                                                       ctypes.c_float(EPS))
        measure(rmsnorm_shard, (2 * rows * HIDDEN + HIDDEN) * 2, "rmsnorm_bf16_8192", count)

        def copy_shard():
            ref = support.Reference(kind)
            ts, td = ref.tensor((rows, 2048), DataType.BF16), ref.tensor((rows, 2048), DataType.BF16)
            ts.view().from_host(bf16((rows, 2048)))
            vs, vd = ts.view(), td.view()
            return ref, lambda: ref.lib.iomref_copy(ref.queue, vs.handle, vd.handle)
        measure(copy_shard, 2 * rows * 2048 * 2, "copy_bf16", count)

        def embedding_shard():
            ref = support.Reference(kind)
            table, ids, out = (ref.tensor((32000, 2048), DataType.BF16), ref.tensor((1, 64), DataType.U32),
                               ref.tensor((64, 2048), DataType.BF16))
            ids.view().from_host(rng.integers(0, 32000, (1, 64)).astype(np.uint32))
            vt, vi, vo = table.view(), ids.view(), out.view()
            return ref, lambda: ref.lib.iomref_embedding(ref.queue, vt.handle, vi.handle, vo.handle)
        measure(embedding_shard, 2 * 64 * 2048 * 2 + 64 * 4, "embedding_decode", count)

        def append_shard():
            ref = support.Reference(kind)
            k, cache = ref.tensor((4, 1, 64), DataType.BF16), ref.tensor((4, 2048, 64), DataType.BF16)
            k.view().from_host(bf16((4, 1, 64)))
            vk, vc = k.view(), cache.view()
            return ref, lambda: ref.lib.iomref_cache_append(ref.queue, vk.handle, vc.handle, 1000)
        measure(append_shard, 2 * 4 * 64 * 2, "cache_append_decode_one_sequence", count)
    return results


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
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f32 accumulate, bf16 storage",
        "data": "synthetic (seeded normal, the large sharded configuration's distributions)",
        "config": {"workload": workload(world), "sample": cpu["sample"],
                   "rows_per_step": cpu["rows_per_step"]},
        "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cpu["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=40)
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
    parser.add_argument("--rows", type=int, default=ROWS,
                        help="rows of the [rows, 8192] tensor; smaller values give the small "
                             "case profiler captures use")
    args = parser.parse_args()
    configure(args.rows)
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
            if not args.no_ops:
                threads = max(1, min(os.cpu_count() or 1, 16))
                try:
                    result["cpu_baseline"]["per_op"] = cpu_per_op(threads)
                except Exception as error:
                    result["cpu_baseline"]["per_op"] = {"error": str(error)}
    restore = getattr(args, "_restore_stdout", None)
    if restore is not None:
        sys.stdout.flush()
        restore()
    if result is not None:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
