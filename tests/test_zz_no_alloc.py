"""The allocation-free sum (b200_sum_f32_static) against the routine path.

Some callers cannot allocate device memory while they run: a stream capture forbids it, a
serving loop cannot afford the synchronisation cudaMalloc implies, a process may have handed
out its whole memory budget already.  For them the library offers one reduction whose scratch
is a fixed array inside its device image.  This test calls it through the C ABI and compares
it with the same sum computed by a compiled routine (b200_compile / b200_link / b200_launch,
whose grid-wide reduction takes its scratch from the routine's allocated slab), twice in a row
with different data so that a stale partial from the first call would show in the second.

Collected last on purpose (the file name sorts after every other test file): a run that stops
at the first failure has then already run everything else.
"""
import numpy as np
import pytest

from ocannl_b200 import backend as bk
from ocannl_b200.low_level import Routine, Seq, Set
from ocannl_b200.workloads import reduce_scope

pytestmark = pytest.mark.gpu


def sum_routine(n: int) -> Routine:
    r = Routine("sum_%d" % n)
    x = r.tn("x", "single", [n], read_only=True)
    out = r.tn("total", "single", [1])
    i = r.sym()
    r.body = Seq([Set(out, (0,), reduce_scope(r, "n_total", "single", [(i, n)], lambda: x[i], op="add"))])
    return r


def test_static_sum_matches_routine_sum_twice(device):
    n = 1_000_003
    ir = sum_routine(n)
    code = bk.Code(ir)
    assert any("grid-wide" in s["note"] for s in code.info()["stages"])      # the scratch-using path
    rt = bk.Context(device).link(code)
    pool, off, _ = rt.context.arrays["x"]
    opool, ooff, _ = rt.context.arrays["total"]
    spool = device.alloc_pool(256)                      # output slot of the static variant
    rng = np.random.default_rng(11)
    for call in range(2):
        x = rng.uniform(0.0, 1.0 + call, n).astype(np.float32)
        rt.context.from_host("x", x)
        rt.run()
        device.sum_f32_static(pool, off, n, spool, 0)
        device.await_()
        want = rt.context.to_host("total")[0]
        got = np.empty(1, np.float32)
        device.to_host(spool, 0, got)
        device.await_()
        exact = float(x.astype(np.float64).sum())
        assert abs(float(want) - exact) <= 1e-5 * exact
        assert abs(float(got[0]) - float(want)) <= 1e-5 * abs(float(want)), (call, got[0], want)
    # a short range (one block) right after a long one: no partial of the long run is read
    x = rng.uniform(0.0, 1.0, n).astype(np.float32)
    rt.context.from_host("x", x)
    device.sum_f32_static(pool, off, 1000, spool, 0)
    device.await_()
    got = np.empty(1, np.float32)
    device.to_host(spool, 0, got)
    device.await_()
    assert abs(float(got[0]) - float(x[:1000].astype(np.float64).sum())) <= 1e-5 * 1000
    rt.free()
    code.free()
    device.free_pool(spool)


def test_static_sum_refuses_what_does_not_fit(device):
    pool = device.alloc_pool(1024)
    with pytest.raises(bk.B200Error) as e:
        device.sum_f32_static(pool, 0, (1 << 26) + 1, pool, 0)
    assert e.value.code == -7 and "capacity" in str(e.value)
    with pytest.raises(bk.B200Error):
        device.sum_f32_static(pool, 0, 1024, pool, 0)          # 4096 bytes do not fit a 1024-byte pool
    # offsets that are not multiples of 4 would be misaligned float accesses on the device:
    # refused on the host, nothing is launched
    for in_off, out_off in ((2, 0), (0, 6), (1, 3)):
        with pytest.raises(bk.B200Error) as e:
            device.sum_f32_static(pool, in_off, 8, pool, out_off)
        assert e.value.code == -1 and "multiples of 4" in str(e.value)
    # an empty range is a sum of nothing
    device.from_host(pool, 0, np.float32([7.0]))
    device.sum_f32_static(pool, 16, 0, pool, 0)
    got = np.empty(1, np.float32)
    device.to_host(pool, 0, got)
    device.await_()
    assert got[0] == 0.0
    device.free_pool(pool)
