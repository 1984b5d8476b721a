"""Hand-built IR of the routines behind the reference's golden generated-C files.

Each function rebuilds, from the reference test program that produced the golden,
the `Low_level` routine the cc backend printed:
  d_fwd      test/operations/top_down_prec.ml      -> top_down_prec.c.expected
  out_fwd    test/operations/zero_out_local_decl.ml -> zero_out_local_decl.c.expected
  where_fwd  test/operations/test_where_precision.ml -> test_where_precision.c.expected
"""
from ocannl_b200.low_level import (Comment, EmbedIndex, For, Routine, Seq, Set, ZeroOut, where)


def d_fwd() -> Routine:
    r = Routine("d_fwd")
    a = r.tn("a", "half", [1])
    b = r.tn("b", "half", [1])
    c = r.tn("c", "bfloat16", [1])
    d = r.tn("d", "bfloat16", [1])
    r.body = Seq([Comment("d fwd"), Set(d, (0,), (a[0] + b[0]) * c[0]), Comment("end")])
    return r


def out_fwd() -> Routine:
    r = Routine("out_fwd")
    r._next_sym = 7
    sparse = r.tn("sparse", "single", [4, 3], mode="local", zero_init=True)
    out = r.tn("out", "single", [4])
    i7 = r.sym()
    r._next_sym = 10
    i10 = r.sym()
    r.body = Seq([
        Comment("out fwd"),
        ZeroOut(sparse),
        For(i7, 0, 3, Set(sparse, (i7, 0), EmbedIndex(i7))),
        For(i10, 0, 3, Set(out, (i10,), sparse[i10, 2] * sparse[i10, 2])),
        Comment("end")])
    return r


def where_fwd() -> Routine:
    r = Routine("where_fwd")
    cond = r.tn("cond_condition", "byte", [1])
    a = r.tn("a_then_val", "half", [1])
    b = r.tn("b_else_val", "bfloat16", [1])
    w = r.tn("where", "single", [1])
    r.body = Seq([Comment("where fwd"), Set(w, (0,), where(cond[0], a[0], b[0])), Comment("end")])
    return r


GOLDEN = {"top_down_prec": d_fwd, "zero_out_local_decl": out_fwd, "test_where_precision": where_fwd}
