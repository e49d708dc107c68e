"""Host-side multi-rank logic on CPU: row sharding and the rank-ordered sum of
squares combine, run as two gloo ranks. The per-rank partials come from the
oracle; the sharded result must equal the oracle on the whole tensor."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from iom_b200.sharding import combine_partials, shard_rows
from iom_b200.tensor import DataType
from support import HostTensor, abi, oracle, random_payload


def test_shard_rows_cover_whole_bands():
    for rows in (1, 15, 16, 17, 100, 8192, 262144):
        for world in (1, 2, 3, 4, 8):
            covered = 0
            for rank in range(world):
                first, count = shard_rows(rows, world, rank)
                assert first == covered or count == 0
                assert first % 16 == 0
                covered += count
                if count and first + count < rows:
                    assert count % 16 == 0
            assert covered == rows
    assert shard_rows(262144, 8, 3) == (3 * 32768, 32768)
    with pytest.raises(ValueError):
        shard_rows(16, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, rows, cols, payload, weight, expected_out, expected_sum, failures):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from iom_b200.sharding import all_gather_sum
        first, count = shard_rows(rows, world, rank)
        # Each rank holds its own self-contained tiled shard and a replicated scale.
        x = HostTensor((count, cols), DataType.BF16)
        x.view().copy_from_host(payload[first:first + count])
        w = HostTensor((1, cols), DataType.BF16)
        w.view().copy_from_host(weight)
        out = HostTensor((count, cols), DataType.BF16)
        assert oracle().iomo_rmsnorm(abi(x.view()), abi(w.view()), abi(out.view()), 1e-6, 0) == 0
        # Row independence: the shard's output equals the rows of the unsharded run.
        got = out.view().copy_to_host().view(np.uint16).reshape(count, cols)
        assert np.array_equal(got, expected_out[first:first + count])
        local = torch.tensor([np.float32(oracle().iomo_sumsq(abi(x.view())))], dtype=torch.float32)
        total = all_gather_sum(local)
        everyone = [torch.empty_like(total.reshape(1)) for _ in range(world)]
        dist.all_gather(everyone, total.reshape(1))
        assert all(torch.equal(everyone[0], t) for t in everyone)      # identical on all ranks
        assert abs(float(total) - expected_sum) <= 1e-6 * expected_sum
        dist.barrier()
        dist.destroy_process_group()
    except Exception as error:  # surfaced in the parent
        failures.put(f"rank {rank}: {error!r}")
        raise


def test_two_rank_sharded_rmsnorm_and_sumsq():
    rows, cols, world = 80, 96, 2
    rng = np.random.default_rng(2)
    payload = random_payload(rng, (rows, cols), DataType.BF16, "normal")
    weight = random_payload(rng, (1, cols), DataType.BF16, "normal")
    x = HostTensor((rows, cols), DataType.BF16)
    x.view().copy_from_host(payload)
    w = HostTensor((1, cols), DataType.BF16)
    w.view().copy_from_host(weight)
    out = HostTensor((rows, cols), DataType.BF16)
    assert oracle().iomo_rmsnorm(abi(x.view()), abi(w.view()), abi(out.view()), 1e-6, 0) == 0
    expected_out = out.view().copy_to_host().view(np.uint16).reshape(rows, cols)
    expected_sum = oracle().iomo_sumsq(abi(x.view()))
    context = mp.get_context("spawn")
    failures = context.Queue()
    port = _free_port()
    procs = [context.Process(target=_rank_main,
                             args=(rank, world, port, rows, cols, payload, weight, expected_out,
                                   expected_sum, failures))
             for rank in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    messages = []
    while not failures.empty():
        messages.append(failures.get())
    assert not messages, messages
    assert all(p.exitcode == 0 for p in procs)


def test_combine_partials_is_rank_ordered_fp32():
    parts = [np.float32(1e8), np.float32(1.0), np.float32(-1e8), np.float32(1.0)]
    assert combine_partials(parts) == np.float32(1.0)      # ((1e8+1)-1e8)+1 in FP32
