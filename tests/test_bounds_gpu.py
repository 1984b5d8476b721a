"""The range-checked build (`bounds=1`): every access a generated kernel makes to a node is compared
with the node's size; an access outside it is skipped and reported, nothing is read or written
outside the node.  Checked kernels must compute what the unchecked ones compute."""
import numpy as np
import pytest

from ocannl_b200 import backend as bk
from ocannl_b200 import workloads as W
from ocannl_b200.low_level import Routine, Seq, Set, loops
from tests.parity import compare, run_device, run_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    return bk.Device(0)


def test_checked_kernels_compute_the_same(device):
    x, y = W.moons_inputs()
    cases = [
        (W.moons_train_step(), dict(W.moons_params(), moons_flat=x, moons_classes=y), [{"i1": 0, "i2": 0}, {"i1": 1, "i2": 1}], 1e-5, 1e-6),
        (W.mlp_train_update(rows=64, dims=(32, 64, 64, 10)),
         dict(W.mlp_params(dims=(32, 64, 64, 10)), **dict(zip(("x", "labels"), W.mlp_inputs(rows=64, in_dim=32)))), [{}], 2e-2, 2e-3),
    ]
    for ir, inputs, statics, rtol, atol in cases:
        want = run_oracle(ir, inputs, statics)
        got, info = run_device(device, ir, inputs, statics, options="bounds=1")
        assert all(s["kind"] in ("generic", "memset") for s in info["stages"]), info
        compare(ir, got, want, rtol=rtol, atol=atol)


def test_an_access_outside_a_node_is_skipped_and_reported(device):
    # y has 8 elements, the loop runs to 12: elements 8 .. 11 do not exist
    r = Routine("overrun")
    x = r.tn("x", "single", [12], read_only=True)
    y = r.tn("y", "single", [8])
    guard = r.tn("guard", "single", [8])       # allocated right behind y: must stay untouched
    (i,) = r.syms(1)
    (j,) = r.syms(1)
    r.body = Seq([loops([(j, 8)], Set(guard, (j,), x[j] * 0.0 + 7.0)), loops([(i, 12)], Set(y, (i,), x[i] + 1.0))])
    code = bk.Code(r, "bounds=1")
    rt = bk.Context(device).link(code)
    rt.context.from_host("x", np.arange(12, dtype=np.float32))
    rt.run()
    with pytest.raises(bk.B200Error) as e:
        device.await_()
    assert "outside the node" in str(e.value) and "element" in str(e.value)
    assert np.array_equal(rt.context.to_host("y"), np.arange(8, dtype=np.float32) + 1.0)
    assert np.array_equal(rt.context.to_host("guard"), np.full(8, 7.0, np.float32))
    rt.free()
    code.free()
    # the device stays usable, and a routine that stays inside its nodes reports nothing
    ok = Routine("in_range")
    a = ok.tn("a", "single", [12], read_only=True)
    b = ok.tn("b", "single", [12])
    (k,) = ok.syms(1)
    ok.body = Seq([loops([(k, 12)], Set(b, (k,), a[k] + 1.0))])
    got, _ = run_device(device, ok, {"a": np.arange(12, dtype=np.float32)}, options="bounds=1")
    assert np.array_equal(got["b"], np.arange(12, dtype=np.float32) + 1.0)
