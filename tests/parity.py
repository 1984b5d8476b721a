"""Shared parity harness: run one routine on the device library and on the CPU oracle
(the restated cc backend) from the same seeded inputs and compare every in-context node."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np

from ocannl_b200 import backend as bk
from ocannl_b200.low_level import Routine
from ocannl_b200.workloads import load
from oracle.run_c import OracleRoutine


def run_oracle(ir: Routine, inputs: Dict[str, np.ndarray], statics: Sequence[Dict[str, int]] = ({},)):
    o = OracleRoutine(ir.to_b200ir())
    bufs = o.buffers()
    for k, v in inputs.items():
        bufs[k][...] = np.asarray(v).reshape(bufs[k].shape)
    for st in statics:
        o.run(bufs, st)
    return bufs


def run_device(device, ir: Routine, inputs: Dict[str, np.ndarray], statics: Sequence[Dict[str, int]] = ({},),
               options: Optional[str] = None, graph: bool = False):
    code = bk.Code(ir, options)
    ctx = bk.Context(device)
    rt = ctx.link(code)
    for k, v in inputs.items():
        rt.context.from_host(k, v)
    if graph:
        rt.use_graph(True)
    for st in statics:
        rt.run(**st)
    device.await_()
    out = {t.ident: rt.context.to_host(t.ident) for t in ir.params()}
    info = code.info()
    rt.free()
    code.free()
    pools = {p for p, _, _ in rt.context.arrays.values()}
    for p in pools:
        device.free_pool(p)
    return out, info


def compare(ir: Routine, got: Dict[str, np.ndarray], want: Dict[str, np.ndarray], rtol: float, atol: float,
            only: Optional[List[str]] = None, exact: Sequence[str] = ()):
    """Asserts |got - want| <= atol + rtol*|want| per element for every in-context node
    (or those in `only`); nodes in `exact` must match bit for bit."""
    worst = {}
    for t in ir.params():
        if only is not None and t.ident not in only:
            continue
        g, w = got[t.ident].reshape(-1), want[t.ident].reshape(-1)
        if t.ident in exact:
            assert np.array_equal(g.view(np.uint8), w.view(np.uint8)), "node %s differs bitwise" % t.ident
            continue
        gf, wf = load(t.prec, g).astype(np.float64), load(t.prec, w).astype(np.float64)
        assert np.all(np.isfinite(gf) == np.isfinite(wf)), "node %s: non-finite mismatch" % t.ident
        fin = np.isfinite(wf)
        err = np.abs(gf[fin] - wf[fin])
        tol = atol + rtol * np.abs(wf[fin])
        bad = err > tol
        worst[t.ident] = float((err / np.maximum(tol, 1e-300)).max()) if err.size else 0.0
        assert not bad.any(), "node %s: %d of %d elements off; worst |err|=%g at want=%g" % (
            t.ident, int(bad.sum()), err.size, float(err[bad].max()), float(wf[fin][bad][np.argmax(err[bad])]))
    return worst
