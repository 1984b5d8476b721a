"""Hand-built IR of the routines behind the reference's golden generated-C files.

Each function rebuilds, from the reference test program that produced the golden,
the `Low_level` routine the cc backend printed:
  d_fwd      test/operations/top_down_prec.ml      -> top_down_prec.c.expected
  out_fwd    test/operations/zero_out_local_decl.ml -> zero_out_local_decl.c.expected
  where_fwd  test/operations/test_where_precision.ml -> test_where_precision.c.expected
  slides_gd_update  the three statements the C listing of
             docs/slides-basics_backprop_training_codegen.md:838-866 prints in full (a
             materialised-accumulate contraction as an `fmaf` nest, `fmaxf(0.0, ...)`, the
             SGD line with its `(float)(0.0001)` constant)
and, for the random-number path, the routine of the IR golden
  n3_fwd     test/operations/n3_fwd_with_prec-unoptimized.ll.expected
(seed 0x2A as constant bits, a counter from the loop index, 2-round threefry, vector uniform
conversion), whose single-precision results the reference prints in
test/operations/test_threefry4x32.ml:37-45.
"""
from ocannl_b200.low_level import (VEC_LENGTH, Affine, Binop, Comment, Const, ConstBits, EmbedIndex, For, Routine, Seq,
                                   Set, SetFromVec, Unop, ZeroOut, fma, un, where)


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


def n3_fwd(prec: str = "half", count: int = 5, variant: str = "light", scalar_too: bool = False) -> Routine:
    """random_seed := 0x2A; n1 := index; bits := seed ^^ n1; n3[len*i ..] := uniform(bits[i])."""
    r = Routine("n3_fwd_" + prec + "_" + variant)
    r._next_sym = 5
    seed = r.tn("random_seed", "uint4x32", [count])
    n1 = r.tn("n1", "uint4x32", [count])
    bits = r.tn("threefry4x32_" + variant, "uint4x32", [count])
    length = VEC_LENGTH[prec]
    n3 = r.tn("n3", prec, [length * count])
    i5, i6, i7, i8 = r.syms(4)
    body = [
        Comment("n3 fwd"),
        For(i5, 0, count - 1, Set(seed, (i5,), ConstBits(0x2A))),
        For(i6, 0, count - 1, Set(n1, (i6,), EmbedIndex(i6))),
        For(i7, 0, count - 1, Set(bits, (i7,), Binop("threefry4x32_" + variant, seed[i7], n1[i7]))),
        For(i8, 0, count - 1, SetFromVec(n3, (Affine(((length, i8),)),), length, bits[i8])),
    ]
    if scalar_too:
        # the one-value form of the conversion (Ops.Uint4x32_to_prec_uniform1)
        first = r.tn("first", prec, [count])
        i9 = r.sym()
        body.append(For(i9, 0, count - 1, Set(first, (i9,), Unop("uint4x32_to_prec_uniform1", bits[i9], prec=prec))))
    body.append(Comment("end"))
    r.body = Seq(body)
    return r


def slides_gd_update() -> Routine:
    r = Routine("scalar_loss_forward_and_gradient_then_gd_update")
    i1 = r.static_sym(80)
    r.static_sym(None)
    b1 = r.tn("b1", "single", [16])
    lr = r.tn("learning_rate", "single", [1])
    flat = r.tn("moons_flat", "single", [80, 10, 2])
    w1 = r.tn("w1", "single", [16, 2])
    w3 = r.tn("w3", "single", [1, 16])
    w3g = r.tn("w3_grad", "single", [1, 16], mode="local", zero_init=True)
    n35 = r.tn("n35", "single", [10, 16], mode="local", zero_init=True)
    relu = r.tn("relu", "single", [10, 16], mode="local")
    r._next_sym = 52
    i52, i53, i54 = r.syms(3)
    r._next_sym = 61
    i61, i62 = r.syms(2)
    r._next_sym = 160
    i160 = r.sym()
    r.body = Seq([
        Comment("scalar_loss forward and gradient update"),
        For(i52, 0, 9, For(i53, 0, 15, For(i54, 0, 1, Set(n35, (i52, i53), fma(w1[i53, i54], flat[i1, i52, i54], n35[i52, i53]))))),
        For(i61, 0, 9, For(i62, 0, 15, Set(relu, (i61, i62), un("relu", b1[i62] + n35[i61, i62])))),
        Comment("w3 param sgd step"),
        For(i160, 0, 15, Set(w3, (0, i160), w3[0, i160] - lr[0] * fma(Const(0.0001), w3[0, i160], w3g[0, i160]))),
        Comment("end"), Comment("end")])
    return r


GOLDEN = {"top_down_prec": d_fwd, "zero_out_local_decl": out_fwd, "test_where_precision": where_fwd}
