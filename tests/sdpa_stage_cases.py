"""The fixtures and known answers of the reference's stage test
(test/cuda/test_cuda_sdpa_nonmatrix.cpp), restated as data so that the oracle (CPU) and the
kernels (GPU) are checked against the same expectations, plus seeded random workloads."""
import numpy as np

from support import HostStages

INF = np.float32(np.inf)


def special_policy_case() -> HostStages:
    """'stages honor logical rows and special policy' (test lines 212-346): planes 2,
    Hq 4, Hkv 2, R 17, C 24, D 8, a 3, L 19; every cell 12345 except plane 0 / head 0."""
    stages = HostStages(2, 4, 2, 17, 24, 8, 3, 19, score_fill=12345.0)
    cells = stages.scores[0, 0]
    for row in range(17):
        cells[row, :stages.visible(row)] = 0.0
    cells[0, :4] = [0.0, 1.0, 2.0, 3.0]
    cells[1, :3] = [INF, 0.0, INF]
    cells[2, :6] = -INF
    cells[3, 1] = np.nan
    cells[4, 0] = -INF
    return stages


def check_special_policy(scores: np.ndarray, probability: np.ndarray) -> None:
    """The CHECK lines 306-339 of the reference test, after scale/mask and softmax."""
    L, R = 19, 17
    assert abs(scores[0, 0, 0, 1] - 1.0 / np.sqrt(8.0)) < 1.0e-6
    assert scores[0, 0, 0, 4] == 12345.0 and scores[0, 0, 0, L] == 12345.0
    p = probability[0, 0]
    assert p[1, 0] == 0x3F00 and p[1, 2] == 0x3F00 and p[1, 1] == 0 and p[1, 4] == 0
    assert (p[2, :6] == 0x7FC0).all() and p[2, 6] == 0
    assert (p[3, :7] == 0x7FC0).all() and p[3, 7] == 0
    assert p[4, 0] == 0
    assert p[0, L] == 0xA5A5 and p[R, 0] == 0xA5A5
    total = (p[0, :4].astype(np.uint32) << 16).view(np.float32).sum()
    assert abs(total - 1.0) < 0.01


def boundary_case(rows: int) -> HostStages:
    """run_boundary_case (test lines 108-209): planes 1, Hq 2, Hkv 1, C 32, D 3, a 1, L 17."""
    stages = HostStages(1, 2, 1, rows, 32, 3, 1, 17)
    for row in range(rows):
        stages.scores[0, :, row, :stages.visible(row)] = 0.0
    return stages


def check_boundary(stages: HostStages, probability: np.ndarray) -> None:
    rows, L = stages.geometry[3], stages.geometry[7]
    for row in range(rows):
        visible = stages.visible(row)
        assert (probability[0, :, row, :visible] != 0).all()
        assert (probability[0, :, row, visible:L] == 0).all()
        assert (probability[0, :, row, L] == 0xA5A5).all()
    assert (probability[0, :, rows:, :] == 0xA5A5).all()


def subnormal_case() -> HostStages:
    """run_subnormal_case (test lines 136-209): a quotient that is a subnormal BF16."""
    stages = HostStages(2, 1, 1, 1, 2, 1, 1, 2)
    stages.scores[0, 0, 0, :2] = [0.0, -92.5]
    stages.scores[1, 0, 0, :2] = [0.0, -93.2]
    return stages


def check_subnormal(probability: np.ndarray) -> None:
    assert probability[0, 0, 0, 1] == 0x0001 and probability[1, 0, 0, 1] == 0x0000


def random_case(seed: int, planes, Hq, Hkv, R, C, D, a, L, specials: bool = True) -> HostStages:
    """Raw QK-like scores N(0, sqrt(D)) in every cell (masked cells too, so that a stage
    that touches them shows), with a few rows carrying NaN, +inf, -inf and zeros."""
    rng = np.random.default_rng(seed)
    stages = HostStages(planes, Hq, Hkv, R, C, D, a, L)
    stages.scores[...] = (rng.standard_normal(stages.scores.shape) * np.sqrt(D)).astype(np.float32)
    if specials:
        flat = stages.scores.reshape(-1, stages.Lp)
        picks = rng.choice(flat.shape[0], size=min(12, flat.shape[0]), replace=False)
        values = [np.nan, INF, -INF, 0.0, -0.0, 1.0e-42, -1.0e-42, 3.0e38]
        for k, row in enumerate(picks):
            columns = rng.choice(stages.Lp, size=min(3, stages.Lp), replace=False)
            flat[row, columns] = values[k % len(values)]
        if flat.shape[0] > 2:
            flat[picks[0] - 1, :] = -INF          # a row of nothing but -inf
    return stages


def bf16_ulp_distance(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Distance in BF16 codes between two arrays of non-negative BF16 values or NaN codes
    (a NaN matches only a NaN)."""
    g, w = got.astype(np.int32), want.astype(np.int32)
    return np.abs(g - w)
