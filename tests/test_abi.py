"""CPU-side checks of the C-ABI library: it loads without a GPU driver, exports every
symbol include/b200.h declares, compiles routines to sm_100a machine code, and reports
errors the way the header says."""
import ctypes
import os
import re

import pytest

from ocannl_b200 import backend as bk
from ocannl_b200 import workloads as W
from ocannl_b200.low_level import Const, Routine, Seq, Set

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    names = declared_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), "libb200.so does not export " + n


def _nvrtc_or_skip():
    try:
        ctypes.CDLL("libnvrtc.so.12")
    except OSError:
        pytest.skip("NVRTC is not installed on this machine")


def test_compile_is_device_independent(built_lib):
    """`compile` may not touch a device (docs/anatomy_of_a_backend.md:97-108): the moons
    training routine compiles to sm_100a kernels on a machine without a GPU."""
    _nvrtc_or_skip()
    fused = bk.Code(W.moons_train_step())
    st = fused.info()["stages"]
    # ~30 tiny stages share ONE single-block launch (a few zero_outs are gone: the first
    # accumulation into a node known to be zero starts from the constant instead)
    assert len(st) == 1 and st[0]["kind"] == "generic" and "fused" in st[0]["note"], st
    assert fused.source().count("__syncthreads()") >= 25
    fused.free()
    code = bk.Code(W.moons_train_step(), options="fuse=0")
    info = code.info()
    kinds = [s["kind"] for s in info["stages"]]
    assert kinds.count("generic") >= 15 and "memset" in kinds
    src = code.source()
    assert "moons_sgd_step_s0" in src and "fmaf(" in src
    # the dW stage keeps the batch loop serial inside each thread (reduction outermost)
    s7 = [s for s in info["stages"] if s["kernel"] == "moons_sgd_step_s7"][0]
    assert "ser=1" in s7["note"]
    code.free()


def test_malformed_ir_is_a_parse_error(built_lib):
    lib = bk.lib()
    h = ctypes.c_void_p()
    for bad in [b"", b"(b200ir 2)", b"(b200ir 1 (name x) (body (frob)))", b"(b200ir 1 (name x) (tnodes (tn 1 a single (0) ctx)) (static) (merge none) (body (noop)))"]:
        rc = lib.b200_compile(b"", bad, ctypes.c_size_t(len(bad)), None, ctypes.byref(h))
        assert rc == -3, (bad, rc, lib.b200_last_error())
        assert lib.b200_last_error()


def test_unknown_node_and_option(built_lib):
    lib = bk.lib()
    h = ctypes.c_void_p()
    ir = b"(b200ir 1 (name x) (tnodes) (static) (merge none) (body (set 9 (0) (const 0x1p+0))))"
    assert lib.b200_compile(b"", ir, ctypes.c_size_t(len(ir)), None, ctypes.byref(h)) == -3
    r = Routine("tiny")
    a = r.tn("a", "single", [1])
    r.body = Seq([Set(a, (0,), Const(1.0))])
    with pytest.raises(bk.B200Error) as e:
        bk.Code(r, options="frobnicate=1")
    assert e.value.code == -1


def test_no_gpu_fails_loudly(built_lib):
    """Without a driver every device entry point fails with B200_E_NO_DEVICE — nothing
    falls back to the CPU."""
    try:
        ctypes.CDLL("libcuda.so.1")
        pytest.skip("a CUDA driver is present")
    except OSError:
        pass
    with pytest.raises(bk.B200Error) as e:
        bk.num_devices()
    assert e.value.code == -2
    with pytest.raises(bk.B200Error):
        bk.Device(0)
