"""Device parity for the operator table, argmax and the reference's printed known answers."""
import numpy as np
import pytest

from ocannl_b200 import workloads as W
from tests import routines as R
from tests.parity import compare, run_device, run_oracle
from tests.test_oracle_golden import einsum_trivia_expected

pytestmark = pytest.mark.gpu

# results that are one of the arguments, a sign flip, a truncation, 0 or 1, or one exactly rounded
# IEEE operation: the same bits on both sides
EXACT = {"u_relu", "u_sat01", "u_neg", "u_trunc", "u_not", "u_sqrt", "u_recip", "b_add", "b_sub", "b_mul", "b_div",
         "b_relu_gate", "b_sat01_gate", "b_lt", "b_eq", "b_ne", "b_or", "b_and", "b_mod", "b_max", "b_min", "b_arg1", "b_arg2",
         "t_where", "t_fma", "t_mul3"}


def _table_inputs(n, prec):
    g = np.random.default_rng(0)
    if prec == "int32":
        x = g.integers(-3, 4, n).astype(np.int32)
        y = (g.integers(1, 4, n) * g.choice([-1, 1], n)).astype(np.int32)
        z = g.integers(-3, 4, n).astype(np.int32)
        y[::4] = np.where(x[::4] == 0, 1, x[::4])      # equal pairs for eq / ne
        return {"x": x, "y": y, "z": z}
    x = g.normal(0, 1.5, n).astype(np.float32)
    y = g.normal(0, 1.5, n).astype(np.float32)
    z = g.normal(0, 1, n).astype(np.float32)
    y[::4] = x[::4]                                     # equal pairs for eq / ne
    x[1::8] = 0                                         # zeros for not / or / and / where
    y[2::8] = 0
    x[3::16] = np.float32([0.25, 0.5, 1.0, 1.5, -0.5, 2.0, 0.999, 1.001] * (n // 128 + 1))[:len(x[3::16])]   # around sat01's edges
    return {k: W.store(prec, v) for k, v in (("x", x), ("y", y), ("z", z))}


@pytest.mark.parametrize("prec", ["single", "double", "bfloat16", "int32"])
@pytest.mark.parametrize("options", [None, "fuse=0 pairs=0"])
def test_operator_table(device, prec, options):
    """Every entry of `Ops.unop` / `binop` / `ternop` (arrayjit/lib/ops.ml:579-630,688-796) against
    the cc backend's spelling of it.  Selections, comparisons and single IEEE operations agree bit
    for bit; libm functions (exp, log, exp2, log2, sin, cos, tanh, pow, 1/sqrt) within the
    precision's pointwise tolerance: rel 1e-5 in single, one unit in the last place of a 16-bit
    result (the device rounds a hardware approximation there)."""
    n = 4096
    ir = R.operator_table(n, prec)
    inputs = _table_inputs(n, prec)
    want = run_oracle(ir, inputs)
    got, _ = run_device(device, ir, inputs, options=options)
    names = [t.ident for t in ir.params() if t.ident not in ("x", "y", "z")]
    if prec == "int32":
        compare(ir, got, want, 0, 0, exact=names)
        return
    exact = [k for k in names if k in EXACT]
    if prec == "bfloat16":
        # a product or quotient of two bf16 values rounds once in both; u_sqrt / u_recip go through
        # a float function and one rounding in both as well
        exact = [k for k in exact if k not in ("u_sqrt", "u_recip")]
    rest = [k for k in names if k not in exact]
    for k in exact:
        g_, w_ = got[k].reshape(-1), want[k].reshape(-1)
        same = (g_ == w_) | (np.isnan(W.load(prec, g_)) & np.isnan(W.load(prec, w_)))
        assert same.all(), (k, np.argwhere(~same)[:4].ravel(), g_[~same][:4], w_[~same][:4])
    rtol, atol = {"single": (1e-5, 1e-6), "double": (1e-12, 1e-13), "bfloat16": (2.0 ** -7, 2.0 ** -9)}[prec]
    if prec == "double":     # the reference's C text calls `tanhf` on doubles too: single-precision accuracy there
        compare(ir, got, want, rtol=1e-5, atol=1e-6, only=["u_tanh"])
        rest = [k for k in rest if k != "u_tanh"]
    compare(ir, got, want, rtol=rtol, atol=atol, only=rest)


@pytest.mark.parametrize("shape", [(1000, 10), (8192, 27), (300, 1000)])
@pytest.mark.parametrize("options", [None, "fuse=0 coop=0"])
def test_argmax_bit_exact(device, shape, options):
    """argmax as `einmax1` + `eq` + index recovery (tensor/operation.ml:583-593): row maxima,
    the one-hot of their positions and the recovered indices agree with the oracle bit for bit, ties
    included (every position equal to the maximum counts, as in the reference)."""
    rows, classes = shape
    x = np.random.default_rng(8).normal(0, 1, shape).astype(np.float32)
    x[::7, 0] = x[::7].max(1)          # ties with the first column: the recovered "index" is then a sum
    ir = R.argmax_rows(rows, classes)
    want = run_oracle(ir, {"scores": x})
    got, _ = run_device(device, ir, {"scores": x}, options=options)
    compare(ir, got, want, 0, 0, exact=["row_max", "is_max", "argmax"])
    plain = np.ones(rows, bool)
    plain[::7] = False
    assert np.array_equal(got["argmax"].reshape(-1)[plain], x.argmax(1).astype(np.float32)[plain])


@pytest.mark.parametrize("which", ["c", "d", "e", "f"])
@pytest.mark.parametrize("options", [None, "fuse=0 coop=0"])
def test_printed_contractions_on_device(device, which, options):
    """test/einsum/einsum_trivia_exec.ml:67-84 on the device: the results print as the reference's."""
    inputs = {"a": R.range_of_shape([2, 4, 3]), "b": R.range_of_shape([2, 5, 4])}
    got, _ = run_device(device, R.einsum_trivia(which), inputs, options=options)
    assert np.array_equal(np.vectorize(R.printed)(got[which]), einsum_trivia_expected(which))


def test_embedding_lookup_known_answers_on_device(device):
    """test/operations/test_one_hot_embedding_lookup.ml: gathered rows; zero rows for an id equal
    to the vocabulary size, a fractional id and -1."""
    C = np.arange(12, dtype=np.float32).reshape(3, 4)
    for ids, rows in (([1, 3, 0], [[1, 5, 9], [3, 7, 11], [0, 4, 8]]), ([1, 4], [[1, 5, 9], [0, 0, 0]]),
                      ([2, 1.5], [[2, 6, 10], [0, 0, 0]]), ([-1, 3], [[0, 0, 0], [3, 7, 11]])):
        got, _ = run_device(device, R.embedding_lookup(len(ids)), {"ids": np.float32(ids), "C": C})
        assert np.array_equal(got["embedded"], np.float32(rows)), (ids, got["embedded"])


@pytest.mark.parametrize("options", [None, "fuse=0"])
def test_operator_table_fp8(device, options):
    """8-bit floats (1-5-2): every operation widens its arguments, works in float and narrows the
    result with the reference's own -- lossy, not idempotent -- conversion
    (arrayjit/lib/builtins.c:643-742), so values travel as codes and every result is compared bit for
    bit.  For the libm functions a result may fall on the other side of a narrowing threshold when
    the device's function differs in its last bit (tanh of a large argument is 1 on one side and
    the float below 1 on the other, and those narrow to different codes): one result in a hundred
    is allowed there -- the inputs are 256 codes, so one deviating argument shows up many times."""
    n = 4096
    ir = R.operator_table(n, "fp8")
    g = np.random.default_rng(11)
    finite = np.array([c for c in range(256) if (c >> 2) & 0x1F != 0x1F], np.uint8)
    inputs = {k: g.choice(finite, n).astype(np.uint8) for k in ("x", "y", "z")}
    inputs["y"][::4] = inputs["x"][::4]
    inputs["x"][1::8] = 0
    want = run_oracle(ir, inputs)
    got, _ = run_device(device, ir, inputs, options=options)
    libm = {"u_exp", "u_log", "u_exp2", "u_log2", "u_sin", "u_cos", "u_tanh", "b_pow", "u_recip_sqrt"}
    for t in ir.params():
        if t.ident in ("x", "y", "z"):
            continue
        same = got[t.ident] == want[t.ident]
        if t.ident in libm:
            assert same.mean() >= 0.99, (t.ident, float(same.mean()))
        else:
            assert same.all(), (t.ident, np.argwhere(~same)[:4].ravel(), got[t.ident][~same][:4], want[t.ident][~same][:4])
