"""Small lowered routines used by the tests only: forms the benchmark workloads do not contain
(function-scope locals, the operator table, argmax, merge-buffer consumers, the reference's own
known-answer programs)."""
from __future__ import annotations

from typing import List

import numpy as np

from ocannl_b200.low_level import (Binop, Const, DeclareLocal, EmbedIndex, For, Get, GetLocal, GetMerge, LocalScope, Routine,
                                    Seq, Set, SetLocal, Ternop, Unop, binop, fma, loops, un, where)
from ocannl_b200.workloads import reduce_scope


# ------------------------------------------------------------------ cross-statement hoisting
def hoisted_top_level(n: int, prec: str = "single") -> Routine:
    """What `hoist_cross_statement_cse` (arrayjit/lib/low_level.ml:2039-2135) leaves when two
    top-level assignments share a reduction: `Declare_local`, the scope's body, then the users
    reading `Get_local` (printed as a function-scope variable, arrayjit/lib/c_syntax.ml:695-704)."""
    r = Routine("hoisted_top_%d_%s" % (n, prec))
    x = r.tn("x", prec, [n], read_only=True)
    a = r.tn("a", "single", [1])
    b = r.tn("b", prec, [1])
    c = r.tn("c", "single", [4])
    vt = r.tn("n_sq", "single", [1], mode="virtual")
    sid = r.scope(vt)
    k = r.sym()
    i = r.sym()
    r.body = Seq([
        DeclareLocal(sid, False),
        SetLocal(sid, Const(0.0, "single")),
        For(k, 0, n - 1, SetLocal(sid, fma(x[k], x[k], GetLocal(sid)))),
        Set(a, (0,), GetLocal(sid) / float(n)),
        Set(b, (0,), un("sqrt", GetLocal(sid) + 1.0)),
        # a loop nest is no hoisting candidate itself, but may follow and read the variable
        For(i, 0, 3, Set(c, (i,), GetLocal(sid) * EmbedIndex(i))),
    ])
    return r


def hoisted_in_loop(rows: int, cols: int) -> Routine:
    """The same sharing between two assignments of one loop body: declaration, body and users
    all stay inside the loop."""
    r = Routine("hoisted_loop_%dx%d" % (rows, cols))
    m = r.tn("m", "single", [rows, cols], read_only=True)
    p = r.tn("p", "single", [rows])
    q = r.tn("q", "single", [rows])
    vt = r.tn("n_row", "single", [1], mode="virtual")
    sid = r.scope(vt)
    i, k = r.syms(2)
    r.body = For(i, 0, rows - 1, Seq([
        DeclareLocal(sid, True),
        For(k, 0, cols - 1, SetLocal(sid, GetLocal(sid) + m[i, k])),
        Set(p, (i,), GetLocal(sid) * 2.0),
        Set(q, (i,), GetLocal(sid) - 1.0),
    ]))
    return r


# ------------------------------------------------------------------ operator table
UNARY = ("relu", "sat01", "exp", "log", "exp2", "log2", "sin", "cos", "sqrt", "recip", "recip_sqrt", "neg", "trunc",
         "tanh", "not")
BINARY = ("add", "sub", "mul", "div", "pow", "relu_gate", "sat01_gate", "lt", "eq", "ne", "or", "and", "mod", "max",
          "min", "arg1", "arg2")


def operator_table(n: int, prec: str = "single") -> Routine:
    """One assignment per entry of `Ops.unop` / `Ops.binop` / `Ops.ternop`
    (arrayjit/lib/ops.ml:579-630,688-796) over the same inputs: `u_<op>[i] := op(x[i])`,
    `b_<op>[i] := op(x[i], y[i])`, where / fma / mul3 with a third input.  `mod` (C `%`) is only
    defined for integer precisions, whose `y` must hold no zero; `log`, `log2`, `sqrt`, `recip_sqrt` read |x| + 0.5."""
    r = Routine("operator_table_%s_%d" % (prec, n))
    integer = prec in ("int32", "uint32", "int64", "byte")     # (fp8 operations are float operations)
    x = r.tn("x", prec, [n], read_only=True)
    y = r.tn("y", prec, [n], read_only=True)
    z = r.tn("z", prec, [n], read_only=True)
    body: List = []
    for op in UNARY:
        if integer and op not in ("relu", "sat01", "neg", "not", "exp2"):
            continue     # the others go through libm in double and back: not meaningful for integers
        out = r.tn("u_" + op, prec, [n])
        i = r.sym()
        arg = x[i]
        if op in ("log", "log2", "sqrt", "recip_sqrt") and not integer:
            arg = binop("max", x[i], un("neg", x[i])) + 0.5
        body.append(For(i, 0, n - 1, Set(out, (i,), Unop(op, arg, prec))))
    for op in BINARY:
        if op == "pow" and integer:
            continue
        if op == "mod" and not integer:
            continue
        out = r.tn("b_" + op, prec, [n])
        i = r.sym()
        lhs, rhs = x[i], y[i]
        if op == "pow":
            lhs = binop("max", x[i], un("neg", x[i])) + 0.5       # positive base
        # (integer division and `%` need non-zero divisors: the caller keeps zeros out of y)
        body.append(For(i, 0, n - 1, Set(out, (i,), Binop(op, lhs, rhs))))
    for op in ("where", "fma", "mul3"):
        out = r.tn("t_" + op, prec, [n])
        i = r.sym()
        body.append(For(i, 0, n - 1, Set(out, (i,), Ternop(op, x[i], y[i], z[i]))))
    r.body = Seq(body)
    return r


# ------------------------------------------------------------------ argmax
def argmax_rows(rows: int, classes: int, prec: str = "single") -> Routine:
    """`argmax` as the reference composes it (tensor/operation.ml:583-593): the row maximum
    `einmax1 "...|v => ...|0"`, a one-hot of the positions equal to it (`eq`), and the index
    recovered as `sum_v onehot * range` — integer work, compared bit for bit."""
    r = Routine("argmax_%dx%d_%s" % (rows, classes, prec))
    x = r.tn("scores", prec, [rows, classes], read_only=True)
    mx = r.tn("row_max", prec, [rows, 1])
    hot = r.tn("is_max", prec, [rows, classes])
    idx = r.tn("argmax", "single", [rows, 1])
    b, v = r.syms(2)
    s1 = loops([(b, rows)], Set(mx, (b, 0), reduce_scope(r, "n_max", prec, [(v, classes)], lambda: x[b, v], op="max")))
    b, v = r.syms(2)
    s2 = loops([(b, rows), (v, classes)], Set(hot, (b, v), binop("eq", x[b, v], mx[b, 0])))
    b, v = r.syms(2)
    s3 = loops([(b, rows)], Set(idx, (b, 0), reduce_scope(
        r, "n_idx", "single", [(v, classes)], lambda: (hot[b, v], EmbedIndex(v)), op="fma")))
    r.body = Seq([s1, s2, s3])
    return r


# ------------------------------------------------------------------ merge buffer
def merge_add(n: int, prec: str = "single") -> Routine:
    """`[%cd a =+ a.merge]` of test/operations/shard_transfer.ml: the destination adds what the
    device's merge buffer holds (`Get_merge_buffer`, arrayjit/lib/low_level.mli:51)."""
    r = Routine("merge_add_%d_%s" % (n, prec))
    a = r.tn("a", prec, [n])
    r.merge_node = a
    i = r.sym()
    r.body = For(i, 0, n - 1, Set(a, (i,), a[i] + GetMerge(a, (i,))))
    return r


# ------------------------------------------------------------------ the reference's printed known answers
def range_of_shape(dims) -> np.ndarray:
    """`TDSL.range_of_shape`: 0, 1, 2, ... in row-major order."""
    return np.arange(int(np.prod(dims)), dtype=np.float32).reshape(dims)


def einsum_trivia(which: str, prec: str = "single") -> Routine:
    """The contractions of test/einsum/einsum_trivia_exec.ml:67-78 over a (2|3->4, stored
    [batch, output, input] = [2, 4, 3]) and b (2|4->5, stored [2, 5, 4]), each a routine output and
    so a materialised accumulate (`zero_out; for lhs axes, contracted axes { t := fma(x, y, t) }`):
      c = b +* "b|h->o; b|i->h => b|i->o" a      c[b, o, i]    = sum_h  b[b, o, h] * a[b, h, i]
      d = a +* "a|i->h; b|h->o => ab|i->o" b     d[a, b, o, i] = sum_h  a[a, h, i] * b[b, o, h]
      e = a +* "b|i->h; b|h->o => i->o" b        e[o, i]       = sum_bh a[b, h, i] * b[b, o, h]
      f = a +* "a|i->h; b|h->o => i->o" b        f[o, i]       = sum_abh a[a, h, i] * b[b, o, h]"""
    r = Routine("einsum_trivia_" + which + "_" + prec)
    a = r.tn("a", prec, [2, 4, 3], read_only=True)
    b = r.tn("b", prec, [2, 5, 4], read_only=True)
    if which == "c":
        t = r.tn("c", "single", [2, 5, 3])
        ib, io, ii, ih = r.syms(4)
        nest = loops([(ib, 2), (io, 5), (ii, 3), (ih, 4)], Set(t, (ib, io, ii), fma(b[ib, io, ih], a[ib, ih, ii], t[ib, io, ii])))
    elif which == "d":
        t = r.tn("d", "single", [2, 2, 5, 3])
        ia, ib, io, ii, ih = r.syms(5)
        nest = loops([(ia, 2), (ib, 2), (io, 5), (ii, 3), (ih, 4)],
                     Set(t, (ia, ib, io, ii), fma(a[ia, ih, ii], b[ib, io, ih], t[ia, ib, io, ii])))
    elif which == "e":
        t = r.tn("e", "single", [5, 3])
        io, ii, ib, ih = r.syms(4)
        nest = loops([(io, 5), (ii, 3), (ib, 2), (ih, 4)], Set(t, (io, ii), fma(a[ib, ih, ii], b[ib, io, ih], t[io, ii])))
    elif which == "f":
        t = r.tn("f", "single", [5, 3])
        io, ii, ia, ib, ih = r.syms(5)
        nest = loops([(io, 5), (ii, 3), (ia, 2), (ib, 2), (ih, 4)],
                     Set(t, (io, ii), fma(a[ia, ih, ii], b[ib, io, ih], t[io, ii])))
    else:
        raise ValueError(which)
    from ocannl_b200.low_level import ZeroOut
    r.body = Seq([ZeroOut(t), nest])
    return r


def printed(x: float) -> str:
    """A number the way the reference's tensor printer shows it in those tables: two decimals,
    from 10 upwards as a mantissa and an exponent (`4.20e+1`, `1.43e+3`); digits beyond the second
    decimal are cut off, not rounded (1606 prints as 1.60e+3)."""
    from decimal import ROUND_DOWN, Decimal
    d = Decimal(repr(float(x)))
    if abs(d) < 10:
        return str(d.quantize(Decimal("0.01"), rounding=ROUND_DOWN))
    e = d.adjusted()
    m = (d.scaleb(-e)).quantize(Decimal("0.01"), rounding=ROUND_DOWN)
    return "%se%s%d" % (m, "+" if e >= 0 else "-", abs(e))


def embedding_lookup(ids_count: int, vocab: int = 4, embed: int = 3, prec: str = "single") -> Routine:
    """test/operations/test_one_hot_embedding_lookup.ml: `emb[b, o] = C[o, ids[b]]`, written as
    a one-hot reduction and rewritten to a guarded gather
    (`rewrite_one_hot_reductions`, arrayjit/lib/low_level.ml:2158-2329): the guard
    `-1 < id && id < vocab && id == trunc(id)` is evaluated in double."""
    from ocannl_b200.low_level import GetDynamic
    from ocannl_b200.workloads import _force
    r = Routine("embedded_fwd_%d" % ids_count)
    ids = r.tn("ids", "single", [ids_count], read_only=True)
    c = r.tn("C", prec, [embed, vocab], read_only=True)
    emb = r.tn("embedded", prec, [ids_count, embed])
    b, o = r.syms(2)
    D = "double"
    idv = lambda: Get(ids, (b,))
    lower = binop("lt", Const(-1.0, D), idv())
    upper = binop("lt", idv(), Const(float(vocab), D))
    integral = binop("eq", idv(), Unop("trunc", idv(), D))
    guard = _force(binop("and", _force(binop("and", _force(lower, D), _force(upper, D)), D), _force(integral, D)), D)
    r.body = loops([(b, ids_count), (o, embed)], Set(emb, (b, o), where(guard, GetDynamic(c, (o, 0), 1, idv()), Const(0.0, prec))))
    return r


# the attention chain lives with the workloads (bench.py's probe runs it too)
from ocannl_b200.workloads import attention, attention_inputs  # noqa: E402,F401
