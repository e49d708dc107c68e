"""CPU: the oracle's attention stage functions against the known answers of the
reference's own stage test, and against an independent numpy evaluation of the softmax
equations on seeded scores."""
import ctypes

import numpy as np
import pytest

from iom_b200.tensor import DataType
from support import HostTensor, abi, bf16_bits_to_f32, oracle
from sdpa_stage_cases import (boundary_case, check_boundary, check_special_policy, check_subnormal,
                              random_case, special_policy_case, subnormal_case)


def test_special_policy_known_answers():
    stages = special_policy_case().scale_mask().softmax()
    check_special_policy(stages.scores, stages.probability)


@pytest.mark.parametrize("rows", [1, 15, 16, 17])
def test_row_boundaries(rows):
    stages = boundary_case(rows).scale_mask().softmax()
    check_boundary(stages, stages.probability)
    # masked and padding scores keep the fill, visible zeros stay +0
    mask = stages.visible_mask()
    assert (stages.scores[0, :, ~mask] == 777.0).all()
    assert (stages.scores[0, :, mask].view(np.uint32) == 0).all()


def test_subnormal_probability_survives():
    check_subnormal(subnormal_case().scale_mask().softmax().probability)


def test_output_canonicalisation_known_answers():
    """Lines 264-270 and 341-345 of the reference test: -0 -> +0, 0x7FFF -> 0x7FC0, 1.0 kept,
    rows past R and tile padding untouched."""
    out = HostTensor((2, 17, 32), DataType.BF16)
    out.storage.view(np.uint16)[:] = 0x3555
    codes = np.full((2, 17, 32), 0x3555, dtype=np.uint16)
    codes[0, 0, :3] = [0x8000, 0x7FFF, 0x3F80]
    codes[1, 16, 31] = 0xFF81
    out.view().copy_from_host(codes)
    before = out.storage.copy()
    assert oracle().iomo_sdpa_canonicalize_output(abi(out.view())) == 0
    want = codes.copy()
    want[0, 0, :3] = [0, 0x7FC0, 0x3F80]
    want[1, 16, 31] = 0x7FC0
    check = HostTensor((2, 17, 32), DataType.BF16)
    check.storage[:] = before
    check.view().copy_from_host(want)
    assert np.array_equal(out.storage, check.storage)      # rows 17..31 of each plane still 0x3555


def test_softmax_against_numpy_float64():
    """Ordinary rows: probabilities within one BF16 step of the FP64 softmax; masked cells +0."""
    stages = random_case(5, 2, 4, 2, 37, 64, 16, 5, 45, specials=False).scale_mask().softmax()
    planes, Hq, _, R, _, _, a, L = stages.geometry
    for row in range(R):
        visible = stages.visible(row)
        s = stages.scores[:, :, row, :visible].astype(np.float64)
        e = np.exp(s - s.max(axis=-1, keepdims=True))
        want = e / e.sum(axis=-1, keepdims=True)
        got = bf16_bits_to_f32(stages.probability[:, :, row, :visible]).astype(np.float64)
        assert np.all(np.abs(got - want) <= want * 2.0 ** -8 + 1e-30)
        assert (stages.probability[:, :, row, visible:L] == 0).all()
    assert (stages.probability[:, :, :, L:] == 0xA5A5).all()


def test_scale_mask_touches_only_visible_cells():
    stages = random_case(6, 1, 2, 1, 20, 40, 7, 3, 21)
    raw = stages.scores.copy()
    stages.scale_mask()
    mask = stages.visible_mask()
    scale = np.float32(1.0) / np.sqrt(np.float32(7.0))
    want = raw[:, :, mask] * scale
    want = np.where(want == 0, np.float32(0.0), want)
    got = stages.scores[:, :, mask]
    assert np.array_equal(got.view(np.uint32), want.astype(np.float32).view(np.uint32))
    assert np.array_equal(stages.scores[:, :, ~mask].view(np.uint32), raw[:, :, ~mask].view(np.uint32))


def test_rejects_bad_geometry():
    bad = special_policy_case()
    request = bad.request()
    request.L = 25                      # L > C
    assert oracle().iomo_sdpa_softmax(ctypes.byref(request)) == 1
    request = bad.request()
    request.Hkv = 3                     # Hq % Hkv != 0
    assert oracle().iomo_sdpa_scale_mask(ctypes.byref(request)) == 1
