"""Seeded random contractions against the oracle: shapes, layouts and epilogues drawn so that the
matcher's branches all occur -- ragged M / N / K, zero to two batch axes, k-major and n-major second
operands, bf16 / half / single (tf32) operands, an epilogue with a bias, a residual and an activation,
outputs in single or 16-bit precision, node offsets that are or are not 16-byte aligned (the reference's
packing).  Every case must run on the tensor-core path and agree with the oracle within the bf16 / tf32
contraction tolerance (rel 2e-2; the absolute part follows sqrt(K), the scale of a sum of K products)."""
import numpy as np
import pytest

from ocannl_b200 import backend as bk
from ocannl_b200 import workloads as W
from ocannl_b200.low_level import Routine, Seq, Set, loops, un
from tests.parity import compare, run_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    return bk.Device(0)


def _case(seed):
    g = np.random.default_rng(seed)
    nb = int(g.integers(0, 3))
    batch = [int(g.integers(2, 4)) for _ in range(nb)]
    m = int(g.choice([64, 128, 200, 256, 333, 520]))
    n = int(g.choice([16, 40, 64, 96, 128, 200, 256, 264]))
    k = int(g.choice([16, 40, 64, 100, 256, 520]))
    prec = str(g.choice(["bfloat16", "bfloat16", "half", "single"]))
    if prec == "single":
        k = (k + 3) // 4 * 4          # operand rows must stay 16-byte aligned for the tensor maps
        n = (n + 3) // 4 * 4
    else:
        k = (k + 7) // 8 * 8
        n = (n + 7) // 8 * 8
    b_nmajor = bool(g.integers(0, 2))
    y_prec = str(g.choice(["single", prec if prec != "single" else "single"]))
    return dict(batch=batch, m=m, n=n, k=k, prec=prec, b_nmajor=b_nmajor, y_prec=y_prec, bias=bool(g.integers(0, 2)),
                residual=bool(g.integers(0, 2)), act=str(g.choice(["none", "relu", "tanh"])), seed=seed)


def _routine(c):
    r = Routine("rand_%d" % c["seed"])
    bt, m, n, k, P = c["batch"], c["m"], c["n"], c["k"], c["prec"]
    a = r.tn("a", P, bt + [m, k], read_only=True)
    b = r.tn("b", P, bt + ([k, n] if c["b_nmajor"] else [n, k]), read_only=True)
    bias = r.tn("bias", c["y_prec"], [n], read_only=True) if c["bias"] else None
    res = r.tn("res", c["y_prec"], bt + [m, n], read_only=True) if c["residual"] else None
    y = r.tn("y", c["y_prec"], bt + [m, n])
    bs = list(r.syms(len(bt)))
    i, j, kk = r.syms(3)
    acc = W.reduce_scope(r, "acc", "single", [(kk, k)],
                         lambda: (a[tuple(bs + [i, kk])], b[tuple(bs + ([kk, j] if c["b_nmajor"] else [j, kk]))]), orig=tuple(bs + [i, j]))
    v = acc
    if bias is not None:
        v = v + bias[j]
    if c["act"] != "none":
        v = un(c["act"], v)
    if res is not None:
        v = v + res[tuple(bs + [i, j])]
    r.body = Seq([loops([(s, e) for s, e in zip(bs, bt)] + [(i, m), (j, n)], Set(y, tuple(bs + [i, j]), v))])
    return r


def _inputs(c, ir):
    g = np.random.default_rng(1000 + c["seed"])
    out = {}
    for t in ir.params():
        if t.read_only:
            scale = 1.0 / np.sqrt(c["k"]) if t.ident == "b" else 1.0
            out[t.ident] = W.store(t.prec, (g.standard_normal(t.dims) * scale).astype(np.float32))
    return out


@pytest.mark.parametrize("seed", list(range(16)))
@pytest.mark.parametrize("packing", ["aligned", "reference"])
def test_random_contraction(device, seed, packing):
    c = _case(seed)
    ir = _routine(c)
    inputs = _inputs(c, ir)
    want = run_oracle(ir, inputs)
    code = bk.Code(ir)
    ctx = bk.Context(device, packing=packing)
    rt = ctx.link(code)
    for name, v in inputs.items():
        rt.context.from_host(name, v)
    rt.run()
    device.await_()
    got = {t.ident: rt.context.to_host(t.ident) for t in ir.params()}
    info = rt.info()
    rt.free()
    code.free()
    for p in {p for p, _, _ in rt.context.arrays.values()}:
        device.free_pool(p)
    flops = 2.0 * c["m"] * c["n"] * c["k"] * float(np.prod(c["batch"])) if c["batch"] else 2.0 * c["m"] * c["n"] * c["k"]
    if packing == "aligned" and flops >= 4.0e6:       # (smaller problems are not worth a tensor-core launch)
        assert info["stages"][0]["kind"] == "gemm", (c, info)
    # sums of K products of magnitude 1 / sqrt(K) have magnitude ~1, plus a bias and a residual of
    # magnitude ~1: the absolute part of the tolerance is 2e-2 of that scale
    compare(ir, got, want, rtol=2e-2, atol=2e-2, only=["y"])
