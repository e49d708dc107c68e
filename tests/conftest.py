"""pytest configuration: markers and import path."""
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
for entry in (str(ROOT), str(ROOT / "tests")):
    if entry not in sys.path:
        sys.path.insert(0, entry)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_sessionstart(session):
    # IOMB_TRACE_SLOW=<seconds>: dump every thread's Python stack periodically,
    # to see where a slow GPU test run spends its time.
    import os
    period = os.environ.get("IOMB_TRACE_SLOW")
    if period:
        import faulthandler
        path = os.environ.get("IOMB_TRACE_FILE", "slow_trace.log")
        session.config._iomb_trace_file = open(path, "w")
        faulthandler.dump_traceback_later(float(period), repeat=True,
                                          file=session.config._iomb_trace_file)
