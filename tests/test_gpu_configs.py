"""The benchmark configurations as stated, on the GPU.

Configuration 1: F32 A[4096,2048] + bias[2048] -> C, values U(-1,1) from seed 0, bit-exact
against the oracle (whole physical storage).

Configuration 5's sharding rule: a [R, 8192] BF16 tensor cut into row shards on 16-row band
boundaries (iom_b200.sharding.shard_rows) gives, shard by shard, exactly the bytes of the
unsharded run, for residual ADD + RMSNorm (eps 1e-6) with a replicated scale row; and the
whole-tensor sum of squares combined from per-shard FP32 partials in rank order is
reproducible bit for bit and within 1e-6 of an FP64 evaluation.
"""
import gc

import numpy as np
import pytest
import torch

from iom_b200.sharding import combine_partials, shard_rows
from iom_b200.tensor import DataType
from iom_b200.device import DeviceMemoryConfig, make_b200_device
from gpu_support import download, run, upload
from support import HostTensor, abi, bf16_bits_to_f32, f32_to_bf16_bits, oracle

pytestmark = pytest.mark.gpu


@pytest.fixture()
def gpu():
    """A device of its own per case: the whole tensor and every shard's operands are live
    together, which the shared 2 GiB arena of the other modules is not sized for."""
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    gc.collect()
    device = make_b200_device(0, DeviceMemoryConfig(4 << 30))
    queue = device.create_ops()
    yield device, queue
    queue.close()


def test_config_1_f32_bias_add_is_bit_exact(gpu):
    device, queue = gpu
    rng = np.random.default_rng(0)
    a_values = rng.uniform(-1.0, 1.0, size=(4096, 2048)).astype(np.float32)
    bias_values = rng.uniform(-1.0, 1.0, size=(1, 2048)).astype(np.float32)
    a = HostTensor((4096, 2048), DataType.F32).poison()
    bias = HostTensor((1, 2048), DataType.F32).poison()
    c = HostTensor((4096, 2048), DataType.F32).poison(0x5A)
    a.view().copy_from_host(a_values)
    bias.view().copy_from_host(bias_values)
    da, db, dc = upload(device, a), upload(device, bias), upload(device, c)
    run(queue, queue.add(da.view(), db.view(), dc.view()))
    assert oracle().iomo_binary(0, abi(a.view()), abi(bias.view()), abi(c.view()), 0) == 0
    assert np.array_equal(download(dc), c.storage)
    # and the logical result is the plain IEEE sum
    got = HostTensor((4096, 2048), DataType.F32, fill=None)
    got.storage[:] = download(dc)
    assert np.array_equal(got.view().copy_to_host().view(np.float32).reshape(4096, 2048),
                          a_values + bias_values)


def sumsq_of(device, queue, tensor) -> np.float32:
    scratch = device.create_workspace(int(device._lib.iomb_sumsq_scratch_bytes()))
    cell = torch.zeros(8, dtype=torch.float32, device=device.torch_device)
    run(queue, queue.sumsq(tensor.view(), scratch.view(), cell.data_ptr()))
    value = np.float32(cell.cpu().numpy()[0])
    scratch.close()
    return value


@pytest.mark.parametrize("rows", [4096, 4000])
def test_config_5_row_shards_equal_the_unsharded_run(gpu, rows):
    device, queue = gpu
    features, eps = 8192, 1e-6
    rng = np.random.default_rng(2)
    x_values = f32_to_bf16_bits(rng.standard_normal((rows, features), dtype=np.float32))
    r_values = f32_to_bf16_bits(rng.standard_normal((rows, features), dtype=np.float32))
    w_values = f32_to_bf16_bits((1.0 + 0.02 * rng.standard_normal((1, features))).astype(np.float32))

    def device_tensor(values, poison=0xA5):
        host = HostTensor(values.shape, DataType.BF16).poison(poison)
        host.view().copy_from_host(values)
        return upload(device, host)

    def step(x_part, r_part):
        dx, dr = device_tensor(x_part), device_tensor(r_part)
        ds = device_tensor(np.zeros_like(x_part), poison=0x11)
        dn = device_tensor(np.zeros_like(x_part), poison=0x22)
        run(queue, queue.add_rmsnorm(dx.view(), dr.view(), dw.view(), ds.view(), dn.view(), eps))
        return download(ds), download(dn), sumsq_of(device, queue, ds)

    dw = device_tensor(w_values)
    whole_sum, whole_out, whole_sumsq = step(x_values, r_values)
    # The sum of squares runs over the stored sum, which is rounded to BF16.
    stored = HostTensor((rows, features), DataType.BF16, fill=None)
    stored.storage[:] = whole_sum
    stored_values = stored.view().copy_to_host().view(np.uint16).reshape(rows, features)
    truth = float(np.sum(bf16_bits_to_f32(stored_values).astype(np.float64) ** 2))
    band_bytes = 16 * features * 2          # one 16-row band of storage
    for world in (2, 4, 8):
        partials = []
        for rank in range(world):
            first, count = shard_rows(rows, world, rank)
            assert first % 16 == 0
            shard_sum, shard_out, partial = step(x_values[first:first + count],
                                                 r_values[first:first + count])
            begin = first // 16 * band_bytes
            # A shard's storage is the matching run of bands of the whole tensor's storage;
            # rows of a ragged last band keep the poison of their own owner, so only whole
            # storage of complete bands and the logical rows of the last one are compared.
            complete = count // 16 * band_bytes
            assert np.array_equal(shard_sum[:complete], whole_sum[begin:begin + complete])
            assert np.array_equal(shard_out[:complete], whole_out[begin:begin + complete])
            if count % 16:
                tail = HostTensor((count, features), DataType.BF16, fill=None)
                full = HostTensor((rows, features), DataType.BF16, fill=None)
                for shard_bytes, whole_bytes in ((shard_sum, whole_sum), (shard_out, whole_out)):
                    tail.storage[:] = shard_bytes
                    full.storage[:] = whole_bytes
                    got = tail.view().copy_to_host().view(np.uint16).reshape(count, features)
                    want = full.view().copy_to_host().view(np.uint16).reshape(rows, features)
                    assert np.array_equal(got, want[first:first + count])
            partials.append(partial)
        combined = combine_partials(partials)
        assert abs(float(combined) - truth) <= 1e-6 * truth
        # the same shards again: the same bits
        again = [step(x_values[f:f + c], r_values[f:f + c])[2]
                 for f, c in (shard_rows(rows, world, k) for k in range(world))]
        assert [p.tobytes() for p in again] == [p.tobytes() for p in partials]
        assert combine_partials(again).tobytes() == combined.tobytes()
    assert abs(float(whole_sumsq) - truth) <= 1e-6 * truth
