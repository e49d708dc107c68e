"""Host-side fault table: arming, one-shot consumption, skip counts (no device)."""
import pytest

from iom_b200.device import SubmissionFaults


def test_fault_table_is_one_shot_and_counts_passages():
    faults = SubmissionFaults()
    assert not faults.take("launch")
    faults.arm("launch")
    assert faults.take("launch")
    assert not faults.take("launch")              # consumed
    faults.arm("complete", skip=2)
    assert [faults.take("complete") for _ in range(4)] == [False, False, True, False]
    faults.arm("record")
    faults.clear()
    assert not faults.take("record")
    with pytest.raises(ValueError):
        faults.arm("explode")
