"""Failure detection without a GPU fault: the failures are made on the host.

  * a stand-in libnccl (tests/fakes/fake_nccl.c) reports an asynchronous error, or never finishes
    from the caller's point of view; `b200_await` must notice while the stream is still busy, abort
    the communicator and return an error, and the device must keep working;
  * a contraction kernel compiled with `-DB200_INJECT_NO_LOADS` (its producer issues no copies, so
    the operands its other warps wait for never arrive) and a wait limit of 20 ms: the waits run
    out, the kernel sets the device status word, frees its tensor memory and returns;
    `b200_await` reports B200_E_DEVICE and the next routine runs normally.  Nothing hangs or
    faults: the wait is bounded by design and no copy or MMA is in flight when it gives up.
"""
import json
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _child(code: str, env: dict, timeout=300):
    e = dict(os.environ, **env)
    e["PYTHONPATH"] = ROOT + os.pathsep + e.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], env=e, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout + r.stderr
    return json.loads(r.stdout.strip().splitlines()[-1])


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("fake") / "libfake_nccl.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", out, os.path.join(ROOT, "tests", "fakes", "fake_nccl.c")], check=True)
    return out


CHILD = """
    import json, os, numpy as np
    from ocannl_b200 import backend as bk, parallel as par
    dev = bk.Device(0)
    ex = par.NcclExchange(dev, 2, 0, par.NcclExchange.unique_id())
    ex.set_timeout(int(os.environ["TIMEOUT_MS"]))
    pool = dev.alloc_pool(1 << 30)
    for _ in range(int(os.environ["BUSY"])):           # keep the stream busy for a while
        dev.memset_zero(pool, 0, 1 << 30)
    out = {}
    try:
        dev.await_()
        out["error"] = None
    except bk.B200Error as e:
        out["error"] = str(e)
        out["code"] = e.code
    # the device still works
    x = np.arange(1024, dtype=np.float32)
    dev.from_host(pool, 0, x)
    y = np.zeros_like(x)
    dev.to_host(pool, 0, y)
    dev.await_()
    out["device_ok"] = bool(np.array_equal(x, y))
    try:
        ex.allreduce(type("R", (), {"grad_range": (pool, 0, 16)})(), False)
        out["comm_usable"] = True
    except bk.B200Error:
        out["comm_usable"] = False
    ex.free()
    print(json.dumps(out))
"""


def test_asynchronous_nccl_error_aborts_the_communicator(fake_nccl, tmp_path):
    log = str(tmp_path / "nccl.log")
    out = _child(CHILD, {"B200_LIBNCCL": fake_nccl, "FAKE_NCCL_LOG": log, "FAKE_NCCL_FAIL_AFTER": "2", "TIMEOUT_MS": "60000",
                         "BUSY": "400"})
    assert out["error"] and "asynchronous error" in out["error"] and out["code"] == 2, out
    assert out["device_ok"] and not out["comm_usable"], out
    calls = open(log).read().split()
    assert calls.count("abort") == 1 and "destroy" not in calls, calls


def test_collective_that_never_finishes_times_out(fake_nccl, tmp_path):
    log = str(tmp_path / "nccl.log")
    out = _child(CHILD, {"B200_LIBNCCL": fake_nccl, "FAKE_NCCL_LOG": log, "TIMEOUT_MS": "5", "BUSY": "2000"})
    assert out["error"] and "did not finish within 5 ms" in out["error"] and out["code"] == -6, out
    assert out["device_ok"] and not out["comm_usable"], out
    assert open(log).read().split().count("abort") == 1


def test_no_timeout_means_a_plain_wait(fake_nccl, tmp_path):
    log = str(tmp_path / "nccl.log")
    out = _child(CHILD, {"B200_LIBNCCL": fake_nccl, "FAKE_NCCL_LOG": log, "FAKE_NCCL_FAIL_AFTER": "0", "TIMEOUT_MS": "0",
                         "BUSY": "10"})
    assert out["error"] is None and out["device_ok"] and out["comm_usable"], out
    assert "abort" not in open(log).read().split()


WAIT_CHILD = """
    import json, os, numpy as np
    from ocannl_b200 import backend as bk, workloads as W
    from tests.parity import run_device, run_oracle
    dev = bk.Device(0)
    ir = W.einsum_gelu(1, 128, 128, 256)            # one tile, four k blocks
    inputs = W.einsum_gelu_inputs(1, 128, 128, 256)
    out = {}
    os.environ["B200_NVRTC_FLAGS"] = "-DB200_WAIT_LIMIT_NS=20000000ull -DB200_INJECT_NO_LOADS"
    try:
        run_device(dev, ir, inputs)
        out["error"] = None
    except bk.B200Error as e:
        out["error"], out["code"] = str(e), e.code
    del os.environ["B200_NVRTC_FLAGS"]
    got, info = run_device(dev, ir, inputs)           # compiled normally: runs and is right
    want = run_oracle(ir, inputs)
    out["kind"] = info["stages"][0]["kind"]
    out["max_err"] = float(np.abs(got["z"] - want["z"]).max())
    print(json.dumps(out))
"""


def test_bounded_wait_runs_out_and_the_device_recovers():
    out = _child(WAIT_CHILD, {})
    assert out["kind"] == "gemm"
    assert out["error"] and out["code"] == -6 and "bounded wait" in out["error"], out
    assert out["max_err"] < 0.05, out
