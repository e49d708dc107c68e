"""The reference's own backend-neutral conformance suites against the B200 backend.

oracle/_ref/b200_reference_suites is tests/reference_suites/b200_suites.cpp compiled with
the reference's shared suite headers (test/backend/backend_conformance_*.hpp, included
from the reference checkout where it lies) and a small stand-in for the doctest framework.
The driver follows test/cuda/test_cuda_conformance.cpp:163-208: reference CPU device,
candidate and foreign B200 devices on the same ordinal, a storage oracle that seeds and
observes whole owners with plain cudaMemcpy. Each case below is one TEST_CASE of the
driver; the binary exits 0 when no CHECK / REQUIRE of the case failed.
"""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

BINARY = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "b200_reference_suites"

CASES = [
    "supported_data_types is the standard 23-entry table",
    "storage and host transfers for every leaf type",
    "storage oracle identifies a perturbed transfer map",
    "storage oracle covers every leaf width and padded shape",
    "asynchronous copies against the CPU reference",
    "copy validation fails before writes and sequences",
    "transfer failures keep metadata and ownership",
    "deferred queue lifetime and stability",
    "queue cap and workspace contract",
    "embedding lookup reference, admission, and lifetime",
    "cache append reference, admission, and lifetime",
    "RMSNorm reference, admission, and lifetime",
    "binary ADD MUL SUB DIV on the real queue",
]


@pytest.mark.parametrize("case", CASES)
def test_reference_suite(case):
    if not BINARY.exists():
        pytest.skip("oracle/_ref/b200_reference_suites is not built (make -C oracle suites)")
    done = subprocess.run([str(BINARY), case], capture_output=True, text=True, timeout=1200)
    tail = "\n".join(done.stderr.splitlines()[-40:])
    assert done.returncode == 0, f"{case}:\n{tail}"
    assert "[ case ]" in done.stderr, "the case name matched nothing"
