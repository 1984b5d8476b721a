"""Pins the CPU oracle to the reference: golden generated C, numeric known answers and the
reference's own builtins.c compiled into oracle/_ref."""
import ctypes
import hashlib
import json
import os

import numpy as np
import pytest

from ocannl_b200 import workloads as W
from oracle.emit_c import Emitter
from oracle.run_c import OracleRoutine
from tests import routines as R
from tests.golden.golden_routines import GOLDEN, n3_fwd, slides_gd_update
from tests.golden.make_cc_golden_digests import main_logic_text, routine_text
from tests.parity import run_oracle

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(os.path.dirname(HERE), "oracle", "_ref")


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_emitter_reproduces_golden_c(name):
    """The emitted routine text equals the reference's golden generated C once whitespace
    is removed (digests made by tests/golden/make_cc_golden_digests.py)."""
    dig = json.load(open(os.path.join(HERE, "golden", "cc_golden_digests.json")))[name]
    text = routine_text(Emitter(GOLDEN[name]().to_b200ir()).function())
    assert len(text) == dig["chars"]
    assert hashlib.sha256(text.encode()).hexdigest() == dig["sha256"]


def test_emitter_reproduces_slides_listing():
    """The C listing of docs/slides-basics_backprop_training_codegen.md: a materialised
    accumulate printed as an `fmaf` loop nest, `fmaxf(0.0, ...)` for relu and the SGD assignment
    with its `(float)(0.0001)` constant -- the statements between `/* Main logic. */` and the end
    of the function (the listing's `...` lines dropped), whitespace removed."""
    dig = json.load(open(os.path.join(HERE, "golden", "cc_golden_digests.json")))["slides_gd_update"]
    text = main_logic_text(Emitter(slides_gd_update().to_b200ir()).function())
    assert len(text) == dig["chars"]
    assert hashlib.sha256(text.encode()).hexdigest() == dig["sha256"]


def einsum_trivia_expected(which):
    """The cells the reference printed for one of the four contractions, as an array of strings in
    the result's memory layout (fixture made by tests/golden/make_einsum_kat.py)."""
    cells = json.load(open(os.path.join(HERE, "golden", "einsum_trivia_kat.json")))[which]["cells"]
    if which == "c":       # 0:2|2:3->1:5 -> [b, o, i]; one block, a column-cell per b
        return np.array([[[cells[0][o][b][i] for i in range(3)] for o in range(5)] for b in range(2)])
    if which == "d":       # 0:2,1:2|3:3->2:5 -> [a, b, o, i]; a block per a, a column-cell per b
        return np.array([[[[cells[a][o][b][i] for i in range(3)] for o in range(5)] for b in range(2)] for a in range(2)])
    return np.array([[cells[0][o][0][i] for i in range(3)] for o in range(5)])   # 1:3->0:5 -> [o, i]


@pytest.mark.parametrize("which", ["c", "d", "e", "f"])
def test_oracle_reproduces_printed_contractions(which):
    """test/einsum/einsum_trivia_exec.ml:67-84: batched, outer-batch and batch-reduced matrix
    products of two `range_of_shape` tensors; the oracle's results print as the reference's did."""
    out = run_oracle(R.einsum_trivia(which), {"a": R.range_of_shape([2, 4, 3]), "b": R.range_of_shape([2, 5, 4])})[which]
    assert np.array_equal(np.vectorize(R.printed)(out), einsum_trivia_expected(which))


def test_oracle_embedding_lookup_known_answers():
    """test/operations/test_one_hot_embedding_lookup.ml: C[o, i] = 4 o + i; ids (1, 3, 0) gather
    rows; an id equal to the vocabulary size and a fractional id give zero rows."""
    C = np.arange(12, dtype=np.float32).reshape(3, 4)
    for ids, rows in (([1, 3, 0], [[1, 5, 9], [3, 7, 11], [0, 4, 8]]), ([1, 4], [[1, 5, 9], [0, 0, 0]]),
                      ([2, 1.5], [[2, 6, 10], [0, 0, 0]]), ([-1, 3], [[0, 0, 0], [3, 7, 11]])):
        out = run_oracle(R.embedding_lookup(len(ids)), {"ids": np.float32(ids), "C": C})["embedded"]
        assert np.array_equal(out, np.float32(rows)), (ids, out)


def test_oracle_function_scope_locals():
    """`Declare_local` + body + `Get_local` users (arrayjit/lib/low_level.ml:2039-2135), at the top
    level of the routine and inside a loop body, against numpy."""
    x = np.random.default_rng(5).normal(0, 1, 1000).astype(np.float32)
    out = run_oracle(R.hoisted_top_level(1000), {"x": x})
    ss = float(np.sum(x.astype(np.float64) ** 2))
    assert abs(out["a"][0] - ss / 1000) < 1e-4 and abs(out["b"][0] - np.sqrt(ss + 1)) < 1e-3
    assert np.allclose(out["c"], ss * np.arange(4), rtol=1e-5)
    m = np.random.default_rng(6).normal(0, 1, (30, 50)).astype(np.float32)
    out = run_oracle(R.hoisted_in_loop(30, 50), {"m": m})
    assert np.allclose(out["p"], 2 * m.sum(1), atol=1e-4) and np.allclose(out["q"], m.sum(1) - 1, atol=1e-4)


def test_oracle_argmax():
    x = np.random.default_rng(8).normal(0, 1, (64, 10)).astype(np.float32)
    out = run_oracle(R.argmax_rows(64, 10), {"scores": x})
    assert np.array_equal(out["argmax"].reshape(-1), x.argmax(1).astype(np.float32))


def test_golden_routines_run():
    # d = bf16((bf16(a) + bf16(b)) * c), one rounding per operation
    o = OracleRoutine(GOLDEN["top_down_prec"]().to_b200ir())
    b = o.buffers()
    b["a"][0], b["b"][0] = 1.5, 2.25
    b["c"][:] = W.f32_to_bf16_bits(np.float32([3.0]))
    o.run(b)
    assert W.bf16_bits_to_f32(b["d"])[0] == 11.25
    o = OracleRoutine(GOLDEN["zero_out_local_decl"]().to_b200ir())
    b = o.buffers()
    b["out"][:] = 7
    o.run(b)
    assert np.array_equal(b["out"], np.zeros(4, np.float32))   # sparse[:, 2] is never written


def test_bf16_known_answers():
    """arrayjit/test/test_numerical_types.expected: 3.14159 -> 0x4049 -> 3.140625; 1e-3 -> 0x3a83."""
    bits = W.f32_to_bf16_bits(np.float32([3.14159, 1e-3, 1.0, -2.5, 0.0]))
    assert [hex(int(x)) for x in bits[:2]] == ["0x4049", "0x3a83"]
    assert W.bf16_bits_to_f32(bits)[0] == 3.140625
    assert list(W.bf16_bits_to_f32(bits)[2:]) == [1.0, -2.5, 0.0]


def _ref_lib():
    p = os.path.join(REF_DIR, "libref_builtins.so")
    if not os.path.exists(p):
        pytest.skip("oracle/_ref not built (needs the reference checkout: make -C oracle)")
    try:
        return ctypes.CDLL(p)
    except OSError as e:      # built with -march=native on another host
        pytest.skip("oracle/_ref does not load here: %s" % e)


class U4(ctypes.Structure):
    _fields_ = [("v", ctypes.c_uint32 * 4)]


def _port_lib(tmp_path_factory=None):
    import subprocess
    src = os.path.join(os.path.dirname(HERE), "oracle", "_build", "port_exports.c")
    os.makedirs(os.path.dirname(src), exist_ok=True)
    so = src[:-2] + ".so"
    with open(src, "w") as f:
        f.write('#include "builtins_port.h"\n'
                'uint16_t p_s2b(float f){return single_to_bfloat16(f);}\n'
                'float p_b2s(uint16_t h){return bfloat16_to_single(h);}\n'
                'uint4x32_t p_light(uint4x32_t k, uint4x32_t c){return arrayjit_threefry4x32_light(k,c);}\n'
                'uint4x32_t p_crypto(uint4x32_t k, uint4x32_t c){return arrayjit_threefry4x32_crypto(k,c);}\n'
                'float p_uni(uint32_t x){return uint32_to_single_uniform(x);}\n'
                'uint4x32_t p_widen(uint32_t x){return uint32_to_uint4x32(x);}\n'
                'uint4x32_t p_widen64(uint64_t x){return uint64_to_uint4x32(x);}\n'
                'uint4x32_t p_widen_d(double x){return double_to_uint4x32(x);}\n'
                'double2_t p_uni_d(uint4x32_t x){return uint4x32_to_double_uniform_vec(x);}\n'
                'uint16x8_t p_uni_bf(uint4x32_t x){return uint4x32_to_bfloat16_uniform_vec(x);}\n'
                'void p_uni_hf(uint4x32_t x, void* out){half8_t r = uint4x32_to_half_uniform_vec(x); memcpy(out, &r, 16);}\n'
                'int32x4_t p_uni_i(uint4x32_t x){return uint4x32_to_int32_uniform_vec(x);}\n'
                'uint16_t p_uni1_bf(uint4x32_t x){return uint4x32_to_bfloat16_uniform(x);}\n'
                'double p_uni1_d(uint4x32_t x){return uint4x32_to_double_uniform(x);}\n'
                'float p_fp8s(uint8_t c){return fp8_to_single(c);}\n'
                'uint8_t p_sfp8(float f){return single_to_fp8(f);}\n'
                'void p_sfp8_many(const float* f, uint8_t* out, int n){for (int i = 0; i < n; ++i) out[i] = single_to_fp8(f[i]);}\n'
                'void p_uni_fp8(uint4x32_t x, void* out){uint8x16_t r = uint4x32_to_fp8_uniform_vec(x); memcpy(out, &r, 16);}\n')
    subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-I", os.path.dirname(os.path.dirname(src)), src, "-o", so, "-lm"],
                   check=True)
    return ctypes.CDLL(so)


def test_port_matches_reference_builtins():
    """The restated helpers agree bit for bit with the reference's builtins.c."""
    ref, port = _ref_lib(), _port_lib()
    ref.single_to_bfloat16.restype = ctypes.c_uint16
    ref.single_to_bfloat16.argtypes = [ctypes.c_float]
    port.p_s2b.restype = ctypes.c_uint16
    port.p_s2b.argtypes = [ctypes.c_float]
    ref.bfloat16_to_single.restype = ctypes.c_float
    ref.bfloat16_to_single.argtypes = [ctypes.c_uint16]
    port.p_b2s.restype = ctypes.c_float
    port.p_b2s.argtypes = [ctypes.c_uint16]
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.normal(0, 1, 2000), rng.normal(0, 1e-30, 200), rng.normal(0, 1e30, 200),
                           [0.0, -0.0, 1.0, 65504.0, 1e-45, 3.14159, 0.001, np.inf, -np.inf]]).astype(np.float32)
    for v in vals:
        assert ref.single_to_bfloat16(float(v)) == port.p_s2b(float(v))
    assert np.array_equal(W.f32_to_bf16_bits(vals), np.array([port.p_s2b(float(v)) for v in vals], np.uint16))
    for h in rng.integers(0, 0x7F80, 500):       # finite positive patterns
        assert ref.bfloat16_to_single(int(h)) == port.p_b2s(int(h))
    for fn_ref, fn_port in (("arrayjit_threefry4x32_light", "p_light"), ("arrayjit_threefry4x32_crypto", "p_crypto")):
        fr, fp = getattr(ref, fn_ref), getattr(port, fn_port)
        fr.restype = fp.restype = U4
        fr.argtypes = fp.argtypes = [U4, U4]
        for _ in range(200):
            k = U4((ctypes.c_uint32 * 4)(*[int(x) for x in rng.integers(0, 2**32, 4)]))
            c = U4((ctypes.c_uint32 * 4)(*[int(x) for x in rng.integers(0, 2**32, 4)]))
            assert list(fr(k, c).v) == list(fp(k, c).v)
    ref.uint32_to_single_uniform.restype = port.p_uni.restype = ctypes.c_float
    ref.uint32_to_single_uniform.argtypes = port.p_uni.argtypes = [ctypes.c_uint32]
    ref.uint32_to_uint4x32.restype = port.p_widen.restype = U4
    ref.uint32_to_uint4x32.argtypes = port.p_widen.argtypes = [ctypes.c_uint32]
    for x in [0, 1, 255, 256, 2**31, 2**32 - 1] + [int(v) for v in rng.integers(0, 2**32, 100)]:
        assert ref.uint32_to_single_uniform(x) == port.p_uni(x)
        assert list(ref.uint32_to_uint4x32(x).v) == list(port.p_widen(x).v)


def test_port_fp8_matches_reference_builtins():
    """The 8-bit float conversions (arrayjit/lib/builtins.c:643-742), bit for bit: every code
    widened, and a sweep of floats narrowed -- every code's own value, the midpoints and
    neighbourhoods between codes, subnormals, overflow, infinities and NaN."""
    ref, port = _ref_lib(), _port_lib()
    for lib_, w, n in ((ref, "fp8_to_single", "single_to_fp8"), (port, "p_fp8s", "p_sfp8")):
        getattr(lib_, w).restype = ctypes.c_float
        getattr(lib_, w).argtypes = [ctypes.c_uint8]
        getattr(lib_, n).restype = ctypes.c_uint8
        getattr(lib_, n).argtypes = [ctypes.c_float]
    wide = []
    for c in range(256):
        a, b = ref.fp8_to_single(c), port.p_fp8s(c)
        assert (np.isnan(a) and np.isnan(b)) or np.float32(a).tobytes() == np.float32(b).tobytes(), c
        wide.append(a)
    fin = np.float32([v for v in wide if np.isfinite(v)])
    rng = np.random.default_rng(3)
    sweep = np.concatenate([fin, fin * np.float32(1.0625), fin * np.float32(0.9375), fin * np.float32(1.125),
                            rng.normal(0, 1, 4000), rng.normal(0, 1e-4, 2000), rng.normal(0, 3e4, 2000),
                            [0.0, -0.0, 1e-8, -1e-8, 57344.0, 61440.0, 65536.0, 1e9, np.inf, -np.inf, np.nan]]).astype(np.float32)
    for v in sweep:
        assert ref.single_to_fp8(float(v)) == port.p_sfp8(float(v)), float(v)
    # the quirk that matters downstream: widening and narrowing again is not the identity
    assert port.p_sfp8(port.p_fp8s(0x3E)) == 0x3D      # 1.5 (mantissa 2) comes back with mantissa 1


def test_port_uniform_forms_match_reference_builtins():
    """Vector and scalar uniform conversions and the 64-bit widenings (builtins.c:345-606)."""
    ref, port = _ref_lib(), _port_lib()

    class D2(ctypes.Structure):
        _fields_ = [("v", ctypes.c_double * 2)]

    class H8(ctypes.Structure):
        _fields_ = [("v", ctypes.c_uint16 * 8)]

    class I4(ctypes.Structure):
        _fields_ = [("v", ctypes.c_int32 * 4)]

    pairs = [("uint4x32_to_double_uniform_vec", "p_uni_d", D2), ("uint4x32_to_bfloat16_uniform_vec", "p_uni_bf", H8),
             ("uint4x32_to_int32_uniform_vec", "p_uni_i", I4),
             ("uint4x32_to_bfloat16_uniform", "p_uni1_bf", ctypes.c_uint16),
             ("uint4x32_to_double_uniform", "p_uni1_d", ctypes.c_double)]
    rng = np.random.default_rng(1)
    cases = [[0, 0, 0, 0], [2**32 - 1] * 4, [0xFFFF, 0x10000, 0x8000, 0x7FFF8000]] + \
        [[int(x) for x in rng.integers(0, 2**32, 4)] for _ in range(300)]
    for nr, npn, rt in pairs:
        fr, fp = getattr(ref, nr), getattr(port, npn)
        fr.restype = fp.restype = rt
        fr.argtypes = fp.argtypes = [U4]
        for w in cases:
            a, b = fr(U4((ctypes.c_uint32 * 4)(*w))), fp(U4((ctypes.c_uint32 * 4)(*w)))
            if hasattr(a, "v"):
                assert bytes(a) == bytes(b), (nr, w)     # bit patterns, whatever the element type
            else:
                assert a == b, (nr, w)
    # eight _Float16 come back in a vector register, which ctypes cannot describe: a shim compiled
    # against the reference library stores them through a pointer
    import subprocess
    shim_c = os.path.join(os.path.dirname(HERE), "oracle", "_build", "ref_half_shim.c")
    with open(shim_c, "w") as f:
        f.write('#include <stdint.h>\n#include <string.h>\ntypedef struct { uint32_t v[4]; } uint4x32_t;\n'
                'typedef struct { _Float16 v[8]; } half8_t;\nextern half8_t uint4x32_to_half_uniform_vec(uint4x32_t);\n'
                'void r_uni_hf(uint4x32_t x, void* out){half8_t r = uint4x32_to_half_uniform_vec(x); memcpy(out, &r, 16);}\n')
    shim_so = shim_c[:-2] + ".so"
    subprocess.run(["gcc", "-O2", "-shared", "-fPIC", shim_c, "-o", shim_so, "-L", REF_DIR, "-lref_builtins",
                    "-Wl,-rpath," + REF_DIR], check=True)
    shim = ctypes.CDLL(shim_so)
    shim.r_uni_hf.argtypes = port.p_uni_hf.argtypes = [U4, ctypes.c_void_p]
    shim.r_uni_hf.restype = port.p_uni_hf.restype = None
    for w in cases:
        a, b = np.zeros(8, np.uint16), np.zeros(8, np.uint16)
        shim.r_uni_hf(U4((ctypes.c_uint32 * 4)(*w)), a.ctypes.data)
        port.p_uni_hf(U4((ctypes.c_uint32 * 4)(*w)), b.ctypes.data)
        assert np.array_equal(a, b), w
    ref.uint64_to_uint4x32.restype = port.p_widen64.restype = U4
    ref.uint64_to_uint4x32.argtypes = port.p_widen64.argtypes = [ctypes.c_uint64]
    ref.double_to_uint4x32.restype = port.p_widen_d.restype = U4
    ref.double_to_uint4x32.argtypes = port.p_widen_d.argtypes = [ctypes.c_double]
    for x in [0, 1, 42, 2**32, 2**64 - 1] + [int(v) for v in rng.integers(0, 2**63, 50)]:
        assert list(ref.uint64_to_uint4x32(x).v) == list(port.p_widen64(x).v)
    for d in [0.0, 42.0, -1.5, 1e300, 3.14159]:
        assert list(ref.double_to_uint4x32(d).v) == list(port.p_widen_d(d).v)


def test_threefry_uniform_known_answers():
    """test/operations/test_threefry4x32.ml:37-45 prints the first five uniform values of the
    default seed against the counters 0, 1, ...: the routine of the IR golden
    n3_fwd_with_prec-unoptimized.ll.expected, run by the oracle, gives the same digits."""
    out = run_oracle(n3_fwd("single", 10, "light", scalar_too=True), {})
    assert ["%.4g" % v for v in out["n3"][:5]] == ["0.4638", "0.7325", "0.5608", "0.5066", "0.5019"]
    assert np.all((out["n3"] >= 0.0) & (out["n3"] < 1.0))
    assert np.array_equal(out["first"], out["n3"][::4])      # the one-value form takes word 0
    # the half golden writes 8 values per counter; every precision stays inside [0, 1)
    for prec in ("half", "bfloat16", "double"):
        o = run_oracle(n3_fwd(prec, 5, "light"), {})["n3"]
        v = W.bf16_bits_to_f32(o) if prec == "bfloat16" else o.astype(np.float64)
        assert v.shape == (5 * (2 if prec == "double" else 8),) and np.all((v >= 0.0) & (v <= 1.0))


def test_oracle_moons_step_matches_float64_model():
    """The hand-lowered training routine computes the model it claims to: three steps through
    the oracle track an independent float64 numpy statement of the same update."""
    ir = W.moons_train_step()
    x, y = W.moons_inputs()
    P = W.moons_params()
    inputs = dict(P, moons_flat=x, moons_classes=y)
    statics = [{"i1": 0, "i2": 0}, {"i1": 1, "i2": 1}, {"i1": 50, "i2": 2}]
    got = run_oracle(ir, inputs, statics)
    Pn, loss = dict(P), None
    for st in statics:
        Pn, loss = W.moons_step_numpy(Pn, x[st["i1"]].astype(np.float64), y[st["i1"]].astype(np.float64), st["i2"])
    for k in P:
        np.testing.assert_allclose(got[k], Pn[k], rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(got["scalar_loss"][0], loss, rtol=2e-5)


@pytest.mark.parametrize("wprec", ["single", "bfloat16"])
def test_oracle_makemore_forward(wprec):
    ir = W.makemore_forward(batch=64, wprec=wprec)
    ids, onehot = W.makemore_inputs(batch=64)
    P = W.makemore_params()
    inputs = {k: W.store(wprec, v) for k, v in P.items()}
    inputs.update(input_batch=ids, target_batch=onehot)
    got = run_oracle(ir, inputs)
    Pq = {k: W.load(wprec, W.store(wprec, v)) for k, v in P.items()}
    loss, logits = W.makemore_forward_numpy(Pq, ids, onehot)
    tol = 1e-5 if wprec == "single" else 3e-2
    np.testing.assert_allclose(got["logits"], logits, rtol=tol, atol=tol)
    np.testing.assert_allclose(got["batch_loss"][0], loss, rtol=tol)
    # out-of-range and fractional ids gather 0 (test/operations/test_one_hot_embedding_lookup.ml)
    ids2 = ids.copy()
    ids2[0, 0], ids2[1, 1], ids2[2, 2] = -1.0, 27.0, 1.5
    got2 = run_oracle(ir, dict(inputs, input_batch=ids2))
    emb = W.load(wprec, got2["embed"])
    assert not emb[0, 0].any() and not emb[1, 1].any() and not emb[2, 2].any() and emb[3].any()
