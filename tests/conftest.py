import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on a B200 box)")


_port = [int(os.environ.get("BFB_TEST_PORT_BASE", "0")) or (20000 + (os.getpid() * 7) % 20000)]


def run_ranks(case, nranks, timeout=240, env=None, expect_fail=False, gpu=False):
    """Runs tests/_worker.py <case> as `nranks` processes wired like torchrun does it and
    returns the list of (returncode, output).  Asserts success unless expect_fail."""
    _port[0] += 1
    procs = []
    for r in range(nranks):
        e = dict(os.environ)
        e.update({"RANK": str(r), "WORLD_SIZE": str(nranks), "LOCAL_RANK": str(r),
                  "LOCAL_WORLD_SIZE": str(nranks), "MASTER_ADDR": "127.0.0.1",
                  "MASTER_PORT": str(_port[0]), "PYTHONPATH": ROOT + os.pathsep + e.get("PYTHONPATH", ""),
                  "OMP_NUM_THREADS": "1"})
        if not gpu:
            e["BLUEFOG_B200_FORCE_CPU"] = "1"
        if env:
            e.update(env)
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "_worker.py"), case],
                                      env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    results = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timeout]"
        results.append((p.returncode, out))
    if not expect_fail:
        for r, (code, out) in enumerate(results):
            assert code == 0, f"rank {r} failed in case {case}:\n{out[-4000:]}"
    return results


@pytest.fixture
def ranks():
    return run_ranks
