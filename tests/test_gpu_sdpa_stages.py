"""GPU parity of the attention stages that are not matrix products
(iomb_sdpa_scale_mask / _softmax / _scale_mask_softmax / _canonicalize_output):

* the known answers of the reference's own stage test;
* bit-identical scores, probabilities and outputs to the REFERENCE'S OWN CUDA stage kernels
  (oracle/_ref/libiomref_sdpa_stages.so, the reference's sdpa_nonmatrix.cu compiled
  unmodified), launched on the same device on copies of the same buffers;
* against the CPU oracle (the C library's expf, as the reference CPU backend uses): the
  scaled scores bit for bit, the probabilities within one BF16 code (the device's and the
  C library's expf differ in their last bits), rarely, and nothing outside the logical cells
  touched;
* the fused stage equals the two launches bit for bit.
"""
import ctypes

import numpy as np
import pytest
import torch

from iom_b200.device import OID_INVALID_ARGUMENT, SdpaStages
from iom_b200.tensor import DataType, TensorSpec
from gpu_support import download, gpu, run, upload  # noqa: F401
from support import HostStages, HostTensor, abi, oracle, sdpa_reference_stages_or_skip
from sdpa_stage_cases import (boundary_case, check_boundary, check_special_policy, check_subnormal,
                              random_case, special_policy_case, subnormal_case)

pytestmark = pytest.mark.gpu


class DeviceStages:
    """Device copy of a HostStages workspace."""

    def __init__(self, device, host: HostStages):
        self.host = host
        planes, Hq, Hkv, R, C, D, a, L = host.geometry
        self.workspace = device.create_workspace(SdpaStages.workspace_bytes(planes, Hq, R, L))
        self.stages = SdpaStages(self.workspace.view(), planes, Hq, Hkv, R, C, D, a, L)
        raw = self.workspace.tensor()
        raw[:host.scores.nbytes].copy_(torch.from_numpy(host.scores.view(np.uint8).reshape(-1).copy()))
        start = self.stages.score_bytes
        raw[start:start + host.probability.nbytes].copy_(
            torch.from_numpy(host.probability.view(np.uint8).reshape(-1).copy()))
        torch.cuda.synchronize()

    def scores(self) -> np.ndarray:
        torch.cuda.synchronize()
        raw = self.workspace.tensor()[:self.host.scores.nbytes].cpu().numpy()
        return raw.view(np.float32).reshape(self.host.scores.shape)

    def probability(self) -> np.ndarray:
        torch.cuda.synchronize()
        start = self.stages.score_bytes
        raw = self.workspace.tensor()[start:start + self.host.probability.nbytes].cpu().numpy()
        return raw.view(np.uint16).reshape(self.host.probability.shape)

    def close(self):
        self.workspace.close()


def same_scores(got: np.ndarray, want: np.ndarray) -> bool:
    """Equal bits, or a NaN on both sides: the device's multiplier returns its own NaN code
    for a NaN operand, and the payload of a NaN score is not part of the result."""
    both_nan = np.isnan(got) & np.isnan(want)
    return bool(np.all((got.view(np.uint32) == want.view(np.uint32)) | both_nan))


def reference_stage(lib, stage, ds: DeviceStages, out_tensor=None, out_view=None):
    """One launch of the reference's own kernel on the device buffers of `ds`."""
    planes, Hq, Hkv, R, C, D, a, L = ds.host.geometry
    u64 = ctypes.c_uint64
    if out_view is None:
        strides, dims, rank = (u64 * 1)(1), (u64 * 1)(planes), 1
        offset = 0
    else:
        lead = out_view.spec.rank - 2
        strides = (u64 * max(lead, 1))(*out_view.plane_strides[:lead])
        dims = (u64 * max(lead, 1))(*out_view.spec.shape[:lead])
        rank, offset = lead, out_view.plane_offset
    status = lib.iomref_sdpa_stage(
        stage, ds.stages.scores_address(), ds.stages.probability_address(),
        out_tensor.storage().data_ptr(), out_tensor.storage_nbytes, offset, strides, rank, dims,
        Hq, Hkv, R, C, D, a, L, None)
    assert status == 0, lib.iomref_sdpa_error().decode()
    torch.cuda.synchronize()


def test_known_answers_of_the_reference_stage_test(gpu):
    device, queue = gpu
    ds = DeviceStages(device, special_policy_case())
    run(queue, queue.sdpa_scale_mask(ds.stages))
    run(queue, queue.sdpa_softmax(ds.stages))
    check_special_policy(ds.scores(), ds.probability())
    ds.close()
    for rows in (1, 15, 16, 17):
        host = boundary_case(rows)
        ds = DeviceStages(device, host)
        run(queue, queue.sdpa_scale_mask(ds.stages))
        run(queue, queue.sdpa_softmax(ds.stages))
        check_boundary(host, ds.probability())
        ds.close()
    ds = DeviceStages(device, subnormal_case())
    run(queue, queue.sdpa_scale_mask_softmax(ds.stages))
    check_subnormal(ds.probability())
    ds.close()


GEOMETRIES = [
    # planes, Hq, Hkv, R, C, D, a, L
    (2, 4, 2, 37, 64, 16, 5, 45),        # L > a + R: every row's prefix ends before L
    (1, 2, 1, 40, 64, 64, 0, 40),        # prefill from an empty cache
    (3, 8, 2, 1, 700, 64, 650, 651),     # decode: one row per head, long prefix
    (1, 3, 3, 33, 1600, 8, 1500, 1533),  # several tiles of 128 tokens per row
    (2, 2, 1, 50, 90, 3, 20, 30),        # L < a + R: late rows all see L tokens
    (1, 1, 1, 16, 16, 1, 0, 16),
    (1, 5, 5, 7, 300, 128, 100, 107),
]


# At least 256 rows per SM of a B200 (37 888) of at most 512 tokens: these run the kernel
# with one lane per row.
MANY_ROWS = [
    (1, 64, 4, 600, 700, 64, 12, 500),     # prefixes up to 500 tokens, 38 400 rows
    (300, 8, 2, 16, 40, 16, 24, 40),       # short rows, many planes
    (2, 148, 37, 130, 200, 8, 3, 77),      # L < a + R, head count not a multiple of 32
]


# Thousands of rows of up to 2048 tokens, fewer or longer than the one-lane-per-row kernel
# takes: many groups per CTA of the grouped kernel (ragged prefixes; L < a + R; decode-like
# single rows per head).
PIPELINED = [
    (1, 32, 4, 100, 1200, 64, 1000, 1100),
    (2, 16, 4, 64, 700, 32, 600, 640),
    (1, 16, 2, 128, 2048, 64, 1920, 2048),
    (1, 16, 4, 128, 300, 16, 100, 228),
    (1, 8, 8, 300, 2048, 64, 0, 300),
    (2000, 1, 1, 1, 2047, 8, 2040, 2041),
]


@pytest.mark.parametrize("geometry", GEOMETRIES + MANY_ROWS + PIPELINED)
def test_stages_against_the_oracle(gpu, geometry):
    device, queue = gpu
    host = random_case(11, *geometry)
    ds = DeviceStages(device, host)
    raw = host.scores.copy()
    run(queue, queue.sdpa_scale_mask(ds.stages))
    host.scale_mask()
    assert same_scores(ds.scores(), host.scores)
    run(queue, queue.sdpa_softmax(ds.stages))
    host.softmax()
    assert same_scores(ds.scores(), host.scores)                   # softmax only reads them
    got, want = ds.probability(), host.probability
    distance = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert distance.max() <= 1, f"probabilities differ by {distance.max()} BF16 codes"
    assert (distance != 0).mean() <= 2e-3
    mask = host.visible_mask()
    planes, Hq, _, R, _, _, a, L = host.geometry
    outside = np.ones(mask.shape, dtype=bool)
    outside[:R, :L] = False
    assert (got[:, :, outside] == 0xA5A5).all()                    # padding rows and tokens >= L
    assert (got[:, :, (~mask) & (~outside)] == 0).all()            # masked cells below L
    assert np.array_equal(raw[:, :, ~mask].view(np.uint32), ds.scores()[:, :, ~mask].view(np.uint32))
    ds.close()


@pytest.mark.parametrize("geometry", GEOMETRIES + MANY_ROWS + PIPELINED)
def test_stages_bit_identical_to_the_reference_kernels(gpu, geometry):
    lib = sdpa_reference_stages_or_skip()
    device, queue = gpu
    host = random_case(12, *geometry)
    planes, Hq, _, R, _, D, _, _ = geometry
    mine, theirs = DeviceStages(device, host), DeviceStages(device, host)
    out = device.create_tensor(TensorSpec((planes, R, Hq * D), DataType.BF16))
    run(queue, queue.sdpa_scale_mask(mine.stages))
    reference_stage(lib, 0, theirs, out)
    assert np.array_equal(mine.scores().view(np.uint32), theirs.scores().view(np.uint32))
    run(queue, queue.sdpa_softmax(mine.stages))
    reference_stage(lib, 1, theirs, out)
    assert np.array_equal(mine.probability(), theirs.probability())
    assert np.array_equal(mine.scores().view(np.uint32), theirs.scores().view(np.uint32))
    for ds in (mine, theirs):
        ds.close()
    out.close()


@pytest.mark.parametrize("keep", [False, True])
@pytest.mark.parametrize("geometry", GEOMETRIES[:5] + MANY_ROWS + PIPELINED)
def test_fused_stage_equals_the_two_launches(gpu, geometry, keep):
    device, queue = gpu
    host = random_case(13, *geometry)
    two, one = DeviceStages(device, host), DeviceStages(device, host)
    run(queue, queue.sdpa_scale_mask(two.stages))
    run(queue, queue.sdpa_softmax(two.stages))
    run(queue, queue.sdpa_scale_mask_softmax(one.stages, keep_scores=keep))
    assert np.array_equal(one.probability(), two.probability())
    expected_scores = two.scores() if keep else host.scores
    assert np.array_equal(one.scores().view(np.uint32), expected_scores.view(np.uint32))
    for ds in (two, one):
        ds.close()


def test_stages_replay_from_a_captured_sequence(gpu):
    """The stage entry points neither allocate nor synchronise: a captured sequence of the fused
    stage and the output canonicalisation replays on new scores with the eager results."""
    from iom_b200.device import OID_CAPTURED
    device, queue = gpu
    geometry = (2, 4, 2, 37, 64, 16, 5, 45)
    first, second = random_case(41, *geometry), random_case(42, *geometry)
    eager, graph = DeviceStages(device, second), DeviceStages(device, first)
    negative_zeros = HostTensor((2, 37, 64), DataType.BF16).poison(0x80)
    negative_zeros.view().copy_from_host(np.full((2, 37, 64), 0x8000, dtype=np.uint16))
    out = upload(device, negative_zeros)
    run(queue, queue.sdpa_scale_mask_softmax(eager.stages))
    with queue.capture() as step:
        assert queue.sdpa_scale_mask_softmax(graph.stages) == OID_CAPTURED
        assert queue.sdpa_canonicalize_output(out.view()) == OID_CAPTURED
    run(queue, step.replay())
    want_first = DeviceStages(device, first)
    run(queue, queue.sdpa_scale_mask_softmax(want_first.stages))
    assert np.array_equal(graph.probability(), want_first.probability())
    # new scores in the same buffers, same recorded launches
    graph.workspace.tensor()[:second.scores.nbytes].copy_(
        torch.from_numpy(second.scores.view(np.uint8).reshape(-1).copy()))
    torch.cuda.synchronize()
    run(queue, step.replay())
    assert np.array_equal(graph.probability(), eager.probability())
    cleaned = HostTensor((2, 37, 64), DataType.BF16).poison(0x80)
    cleaned.view().copy_from_host(np.zeros((2, 37, 64), dtype=np.uint16))
    assert np.array_equal(download(out), cleaned.storage)      # -0 became +0, padding untouched
    for ds in (eager, graph, want_first):
        ds.close()
    out.close()


def special_codes(rng, shape):
    codes = rng.integers(0, 65536, size=shape, dtype=np.uint16)
    flat = codes.reshape(-1)
    picks = rng.choice(flat.size, size=max(4, flat.size // 6), replace=False)
    flat[picks] = rng.choice(np.array([0x8000, 0x0000, 0x7FFF, 0xFFFF, 0x7F81, 0xFF80, 0x7F80, 0x0001,
                                       0x8001], dtype=np.uint16), size=picks.size)
    return codes


@pytest.mark.parametrize("shape", [(2, 17, 32), (1, 1, 64), (3, 2, 33, 40), (130, 2048), (5, 16, 7),
                                   (3, 32, 64), (144, 2048), (2, 3, 16, 16)])
def test_output_canonicalisation_against_the_oracle_and_the_reference(gpu, shape):
    device, queue = gpu
    rng = np.random.default_rng(21)
    host = HostTensor(shape, DataType.BF16).poison(0x80)            # padding 0x8080: a value the
    host.view().copy_from_host(special_codes(rng, shape))            # stage would change if it
    mine = upload(device, host)                                      # touched it
    run(queue, queue.sdpa_canonicalize_output(mine.view()))
    assert oracle().iomo_sdpa_canonicalize_output(abi(host.view())) == 0
    assert np.array_equal(download(mine), host.storage)
    mine.close()


def test_output_canonicalisation_of_a_strided_view_matches_the_reference_kernel(gpu):
    lib = sdpa_reference_stages_or_skip()
    device, queue = gpu
    rng = np.random.default_rng(22)
    host = HostTensor((4, 6, 19, 48), DataType.BF16).poison(0x80)
    host.view().copy_from_host(special_codes(rng, (4, 6, 19, 48)))
    mine, theirs = upload(device, host), upload(device, host)
    window = mine.view().slice(0, 1, 2).slice(1, 0, 3, 2)           # planes (1..2, {0,2,4})
    run(queue, queue.sdpa_canonicalize_output(window))
    # the reference request: Hq*D = 48 as 3 heads of 16, R = 19
    stage_host = HostStages(6, 3, 3, 19, 32, 16, 0, 19)
    ds = DeviceStages(device, stage_host)
    their_window = theirs.view().slice(0, 1, 2).slice(1, 0, 3, 2)
    reference_stage(lib, 2, ds, theirs, their_window)
    assert np.array_equal(download(mine), download(theirs))
    assert oracle().iomo_sdpa_canonicalize_output(abi(host.view().slice(0, 1, 2).slice(1, 0, 3, 2))) == 0
    assert np.array_equal(download(mine), host.storage)
    ds.close()
    mine.close()
    theirs.close()


def test_rejections(gpu):
    device, queue = gpu
    workspace = device.create_workspace(SdpaStages.workspace_bytes(1, 2, 16, 16))
    good = SdpaStages(workspace.view(), 1, 2, 1, 16, 16, 4, 0, 16)
    for field, value in (("L", 17), ("a", 16), ("R", 0), ("Hkv", 3), ("D", 0)):
        bad = SdpaStages(workspace.view(), 1, 2, 1, 16, 16, 4, 0, 16)
        setattr(bad, field, value)
        assert queue.sdpa_softmax(bad) == OID_INVALID_ARGUMENT, field
        assert queue.sdpa_scale_mask(bad) == OID_INVALID_ARGUMENT, field
    with pytest.raises(ValueError):
        SdpaStages(workspace.view(), 2, 2, 1, 16, 16, 4, 0, 16)      # workspace too small
    run(queue, queue.sdpa_scale_mask_softmax(good))
    f32 = device.create_tensor(TensorSpec((16, 32), DataType.F32))
    assert queue.sdpa_canonicalize_output(f32.view()) < 0
    f32.close()
    workspace.close()

