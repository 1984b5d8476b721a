"""CPU ORACLE — test infrastructure only, never part of the shipped path.

A restatement of how the reference's `cc` backend turns a lowered routine into
C: it parses the b200ir text of a routine (an independent parser: nothing is
shared with the device library) and prints the C function that
`C_syntax.compile_proc` would print for the same `Low_level.optimized`.

Rules restated, by authority:
  * statements, loops, offsets, local scopes, parameters, local arrays:
    arrayjit/lib/c_syntax.ml:367-379 (offsets), :441-704 (pp_ll),
    :706-855 (pp_scalar), :1021-1210 (compile_proc);
  * operator spellings, type names, precision conversions:
    arrayjit/lib/ops.ml:324-337, :579-630, :688-773, :784-796, :798-863;
  * bf16 / half / fp8 arithmetic done in float with one rounding per op:
    arrayjit/lib/cc_backend.ml:169-322;
  * index printing: arrayjit/lib/indexing.ml:454-476.

Parity pin: `tests/test_oracle_golden.py` checks the emitted function text,
whitespace removed, against the reference's golden generated C
(test/operations/top_down_prec.c.expected, zero_out_local_decl.c.expected,
test_where_precision.c.expected) through committed SHA-256 digests, and the
numeric helpers in `oracle/builtins_port.h` against the reference's own
builtins.c compiled into oracle/_ref.  Pretty-printer line breaking is not
reproduced (it has no effect on the arithmetic).
"""
from __future__ import annotations

import math
import re
from typing import Dict, List, Tuple

# ------------------------------------------------------------- S-expressions
_TOK = re.compile(r'\s*(\(|\)|"(?:[^"\\]|\\.)*"|[^\s()"]+)')


def parse_sexp(text: str):
    pos, stack, cur = 0, [], []
    text = text.strip()
    while pos < len(text):
        m = _TOK.match(text, pos)
        if not m:
            break
        pos = m.end()
        t = m.group(1)
        if t == "(":
            stack.append(cur)
            cur = []
        elif t == ")":
            done = cur
            cur = stack.pop()
            cur.append(done)
        elif t[0] == '"':
            cur.append(("str", t[1:-1].replace('\\"', '"').replace("\\\\", "\\")))
        else:
            cur.append(t)
    assert not stack, "unbalanced b200ir"
    return cur[0]


# ----------------------------------------------------------------- tables
INT_PRECS = ("byte", "uint16", "int32", "uint32", "int64", "uint64", "fp8")
DOUBLEISH = ("double",) + INT_PRECS

C_TYPE = {"byte": "unsigned char", "uint16": "unsigned short", "int32": "int",
          "uint32": "uint32_t", "int64": "long long", "uint64": "uint64_t",
          "uint4x32": "uint4x32_t", "half": "HALF_T", "bfloat16": "unsigned short",
          "fp8": "unsigned char", "single": "float", "double": "double"}


def convert(frm: str, to: str) -> Tuple[str, str]:
    """Ops.c_convert_precision (ops.ml:798-863)."""
    if frm == to:
        return "", ""
    ints = ("byte", "uint16", "int32", "uint32", "int64", "uint64")
    table = {
        ("bfloat16", "single"): ("bfloat16_to_single(", ")"),
        ("single", "bfloat16"): ("single_to_bfloat16(", ")"),
        ("bfloat16", "double"): ("(double)bfloat16_to_single(", ")"),
        ("double", "bfloat16"): ("single_to_bfloat16((float)", ")"),
        ("fp8", "single"): ("fp8_to_single(", ")"),
        ("single", "fp8"): ("single_to_fp8(", ")"),
        ("fp8", "double"): ("(double)fp8_to_single(", ")"),
        ("double", "fp8"): ("single_to_fp8((float)", ")"),
        ("bfloat16", "half"): ("FLOAT_TO_HALF(bfloat16_to_single(", "))"),
        ("half", "bfloat16"): ("single_to_bfloat16(HALF_TO_FLOAT(", "))"),
        ("fp8", "half"): ("FLOAT_TO_HALF(fp8_to_single(", "))"),
        ("half", "fp8"): ("single_to_fp8(HALF_TO_FLOAT(", "))"),
        ("bfloat16", "fp8"): ("single_to_fp8(bfloat16_to_single(", "))"),
        ("fp8", "bfloat16"): ("single_to_bfloat16(fp8_to_single(", "))"),
        ("half", "single"): ("HALF_TO_FLOAT(", ")"),
        ("single", "half"): ("FLOAT_TO_HALF(", ")"),
        ("half", "double"): ("(double)HALF_TO_FLOAT(", ")"),
        ("double", "half"): ("FLOAT_TO_HALF((float)", ")"),
    }
    if (frm, to) in table:
        return table[(frm, to)]
    if frm == "bfloat16" and to in ints:
        return "(" + C_TYPE[to] + ")bfloat16_to_single(", ")"
    if frm in ints and to == "bfloat16":
        return "single_to_bfloat16((float)", ")"
    if frm == "fp8" and to in ints:
        return "(" + C_TYPE[to] + ")fp8_to_single(", ")"
    if frm in ints and to == "fp8":
        return "single_to_fp8((float)", ")"
    if frm == "half" and to in ints:
        return "(" + C_TYPE[to] + ")HALF_TO_FLOAT(", ")"
    if frm in ints and to == "half":
        return "FLOAT_TO_HALF((float)", ")"
    if frm == "uint4x32":
        return "uint4x32_to_" + to + "(", ")"
    if to == "uint4x32":
        return frm + "_to_uint4x32(", ")"
    return "(" + C_TYPE[to] + ")(", ")"


def binop_syntax(prec: str, op: str):
    """Ops.binop_c_syntax (ops.ml:579-630)."""
    if op in ("add", "sub", "mul", "div"):
        return "(", {"add": " +", "sub": " -", "mul": " *", "div": " /"}[op], ")"
    if op == "pow":
        return ("pow(", ",", ")") if prec == "double" else ("powf(", ",", ")")
    if op == "relu_gate":
        return ("(", " > 0 ?", " : 0)") if prec in INT_PRECS else ("(", " > 0.0 ?", " : 0.0)")
    if op == "sat01_gate":
        if prec in INT_PRECS:
            return "(abs(", " ) > 0 ? 0 : (", "))"
        if prec == "single":
            return "(fabsf(floorf(", ")) > 0.0 ? 0.0 : (", "))"
        return "(fabs(floor(", ")) > 0.0 ? 0.0 : (", "))"
    if op == "max":
        return ("fmax(", ",", ")") if prec in DOUBLEISH else ("fmaxf(", ",", ")")
    if op == "min":
        return ("fmin(", ",", ")") if prec in DOUBLEISH else ("fminf(", ",", ")")
    if op in ("threefry4x32_crypto", "threefry4x32_light"):
        return "arrayjit_" + op + "(", ",", ")"      # ops.ml:627-630
    simple = {"mod": " %", "lt": " <", "eq": " ==", "ne": " !=", "or": " ||", "and": " &&"}
    return "(", simple[op], ")"


def unop_syntax(prec: str, op: str):
    """Ops.unop_c_syntax (ops.ml:688-773)."""
    fmax = "fmax" if prec in DOUBLEISH else "fmaxf"
    fmin = "fmin" if prec in DOUBLEISH else "fminf"
    if op == "id":
        return "", ""
    if op == "relu":
        return ("fmax(0, ", ")") if prec in INT_PRECS else (fmax + "(0.0, ", ")")
    if op == "sat01":
        if prec in INT_PRECS:
            return "fmax(0, fmin(1, ", "))"
        return fmax + "(0.0, " + fmin + "(1.0, ", "))"
    libm = {"exp": "exp", "log": "log", "exp2": "exp2", "log2": "log2", "sin": "sin",
            "cos": "cos", "sqrt": "sqrt"}
    if op in libm:
        return (libm[op] + ("(" if prec in DOUBLEISH else "f(")), ")"
    if op == "recip":
        return "(1.0 / (", "))"
    if op == "recip_sqrt":
        return ("(1.0 / sqrt(", "))") if prec == "double" else ("(1.0 / sqrtf(", "))")
    if op == "neg":
        return "(-(", "))"
    if op == "trunc":
        return ("trunc(", ")") if prec == "double" else ("truncf(", ")")
    if op == "tanh":
        return "tanhf(", ")"
    if op == "not":
        return "(", " == 0.0 ? 1.0 : 0.0)"
    if op == "uint4x32_to_prec_uniform1":
        return "uint4x32_to_" + prec + "_uniform(", ")"   # ops.ml:771-773
    raise ValueError(op)


def ternop_syntax(prec: str, op: str):
    """Ops.ternop_c_syntax (ops.ml:784-796)."""
    if op == "where":
        if prec in INT_PRECS:
            return "((", ") != 0 ? (", ") : (", "))"
        return "((", ") != 0.0 ? (", ") : (", "))"
    if op == "fma":
        return ("fma(", ",", ",", ")") if prec in DOUBLEISH else ("fmaf(", ",", ",", ")")
    return "((", ") * (", ") * (", "))"


# Ops.c_vec_typ_of_prec (ops.ml:339-351)
VEC_TYPE = {("single", 4): "float4_t", ("double", 2): "double2_t", ("int32", 4): "int32x4_t",
            ("int64", 2): "int64x2_t", ("uint16", 8): "uint16x8_t", ("bfloat16", 8): "uint16x8_t",
            ("half", 8): "half8_t"}

# cc_backend.ml:169-322 — low-precision results are computed in float.
_LOWP = {"bfloat16": ("bfloat16_to_single(", "single_to_bfloat16("),
         "half": ("HALF_TO_FP(", "FP_TO_HALF("),
         "fp8": ("fp8_to_single(", "single_to_fp8(")}


# ------------------------------------------------------------------ emitter
class Emitter:
    def __init__(self, ir_text: str, large_models: bool = False):
        root = parse_sexp(ir_text)
        assert root[0] == "b200ir" and root[1] == "1", "not b200ir version 1"
        sect = {s[0]: s[1:] for s in root[2:]}
        self.name = sect["name"][0]
        self.tn: Dict[int, dict] = {}
        self.order: List[int] = []
        for t in sect["tnodes"]:
            tid = int(t[1])
            self.tn[tid] = dict(id=tid, ident=t[2], prec=t[3], dims=[int(d) for d in t[4]],
                                mode=t[5], zero_init="zero_init" in t[6:],
                                read_only="read_only" in t[6:])
            self.order.append(tid)
        self.static = [(s[0], None if s[1] == "none" else int(s[1])) for s in sect["static"]]
        m = sect["merge"][0]
        self.merge = None if m == "none" else int(m)
        self.body = sect["body"][0]
        self.idx_t = "uint64_t" if large_models else "uint32_t"
        self.zero_out_seen = set()

    # -- indices (indexing.ml:454-476, c_syntax.ml:367-379)
    def axis(self, i) -> str:
        if isinstance(i, list):
            assert i[0] == "affine"
            off = int(i[1])
            terms = [(s if int(c) == 1 else "%d*%s" % (int(c), s)) for c, s in i[2:]]
            if off > 0:
                terms.append(str(off))
            elif off < 0:
                terms.append("-%d" % -off)
            return "+".join(terms) if terms else "0"
        if i == "sub_axis":
            return ""
        return i

    def offset(self, idcs, dims, dyn_axis=-1, dyn_doc="") -> str:
        if not idcs:
            return "0"
        ax = lambda k: dyn_doc if k == dyn_axis else self.axis(idcs[k])
        doc = ax(0)
        for k in range(1, len(idcs)):
            d = ax(k)
            if doc == "":
                doc = d
            elif d == "":
                doc = "(%s) * %d" % (doc, dims[k])
            else:
                doc = "(%s) * %d + %s" % (doc, dims[k], d)
        return doc

    def scope_name(self, sid, tid) -> str:
        return "v%s_%s" % (sid, self.tn[int(tid)]["ident"])

    # -- operator wrappers with the cc low-precision rule
    def _binop(self, prec, op, v1, v2):
        if prec in _LOWP:
            up, down = _LOWP[prec]
            p, i, s = binop_syntax("single", op)
            return "%s%s%s%s)%s %s%s)%s)" % (down, p, up, v1, i, up, v2, s)
        p, i, s = binop_syntax(prec, op)
        return "%s%s%s %s%s" % (p, v1, i, v2, s)

    def _unop(self, prec, op, v):
        if prec in _LOWP:
            up, down = _LOWP[prec]
            p, s = unop_syntax("single", op)
            return "%s%s%s%s)%s)" % (down, p, up, v, s)
        p, s = unop_syntax(prec, op)
        return p + v + s

    def _ternop(self, prec, op, v1, v2, v3):
        if prec in _LOWP:
            up, down = _LOWP[prec]
            p, i1, i2, s = ternop_syntax("single", op)
            return "%s%s%s%s)%s %s%s)%s %s%s)%s)" % (down, p, up, v1, i1, up, v2, i2, up, v3, s)
        p, i1, i2, s = ternop_syntax(prec, op)
        return "%s%s%s %s%s %s%s" % (p, v1, i1, v2, i2, v3, s)

    # -- Low_level.reads_scope_before_set (low_level.ml:1998-2037): is the local read before
    #    the first definitely executed set?  Decides the "= 0" initialiser of a scope.
    def reads_before_set(self, sid, tid, body) -> bool:
        def is_target(a, b):
            return a == sid and b == tid

        def sc_reads(e) -> bool:
            k = e[0]
            if k == "get_local":
                return is_target(e[1], e[2])
            if k == "scope":
                return st_reads(e[3])
            if k == "get_dyn":
                return sc_reads(e[4][0])
            if k in ("tern", "bin", "un"):
                return any(sc_reads(a[0]) for a in e[2:])
            return False

        def st_reads(s) -> bool:
            k = s[0]
            if k == "seq":
                return any(st_reads(x) for x in s[1:])
            if k == "for":
                return st_reads(s[4])
            if k in ("set", "set_local"):
                return sc_reads(s[3])
            return False

        def scan(s) -> str:
            k = s[0]
            if k == "set":
                return "read" if sc_reads(s[3]) else "neither"
            if k == "set_local":
                if sc_reads(s[3]):
                    return "read"
                return "written" if is_target(s[1], s[2]) else "neither"
            if k == "seq":
                for x in s[1:]:
                    r = scan(x)
                    if r != "neither":
                        return r
                return "neither"
            if k == "for":
                r = scan(s[4])
                if r == "written":
                    return "written" if int(s[2]) <= int(s[3]) else "neither"
                return r
            return "neither"

        return scan(body) != "written"

    # -- scalars (c_syntax.ml:706-855): returns (local definitions, expression)
    def scalar(self, prec: str, e) -> Tuple[List[Tuple[int, str]], str]:
        k = e[0]
        if k == "scope":
            sid, tid, body = e[1], int(e[2]), e[3]
            sprec = self.tn[tid]["prec"]
            init = ""
            if self.reads_before_set(sid, e[2], body):
                p, s = convert("int32", sprec)
                init = " = " + p + "0" + s
            decl = "%s %s%s;" % (C_TYPE[sprec], self.scope_name(sid, tid), init)
            body_doc = self.stmt(body, in_loop=True)
            p, s = convert(sprec, prec)
            return [(int(sid), decl + "\n" + body_doc)], p + self.scope_name(sid, tid) + s
        if k == "get_local":
            p, s = convert(self.tn[int(e[2])]["prec"], prec)
            return [], p + self.scope_name(e[1], e[2]) + s
        if k in ("get", "get_merge"):
            t = self.tn[int(e[1])]
            p, s = convert(t["prec"], prec)
            name = "merge_buffer" if k == "get_merge" else t["ident"]
            return [], "%s%s[%s]%s" % (p, name, self.offset(e[2], t["dims"]), s)
        if k == "get_dyn":
            t = self.tn[int(e[1])]
            p, s = convert(t["prec"], prec)
            defs, dyn = self.scalar(e[4][1], e[4][0])
            dyn_doc = "((%s)(%s))" % (self.idx_t, dyn)
            off = self.offset(e[2], t["dims"], int(e[3]), dyn_doc)
            return defs, "%s%s[%s]%s" % (p, t["ident"], off, s)
        if k == "const":
            a = e[1]
            p, s = convert("double", prec)
            if a == "inf":
                c, neg = "INFINITY", False
            elif a == "-inf":
                c, neg = "(-INFINITY)", False
            elif a == "nan":
                c, neg = "NAN", False
            else:
                v = float.fromhex(a)
                c, neg = "%.16g" % v, v < 0.0
            if p == "" and neg:
                return [], "(" + c + ")" + s
            return [], p + c + s
        if k == "const_bits":
            p, s = convert("int64", prec)
            return [], "%s%sLL%s" % (p, e[1], s)
        if k == "idx":
            p, s = convert("uint64" if self.idx_t == "uint64_t" else "uint32", prec)
            d = self.axis(e[1]) or "0"
            return [], p + d + s
        if k == "bin":
            op = e[1]
            if op == "arg1":
                return self.scalar(prec, e[2][0])
            if op == "arg2":
                return self.scalar(prec, e[3][0])
            d1, v1 = self.scalar(prec, e[2][0])
            d2, v2 = self.scalar(prec, e[3][0])
            return d1 + d2, self._binop(prec, op, v1, v2)
        if k == "un":
            if e[1] == "uint4x32_to_prec_uniform1":   # not homogeneous: ops.ml:955-958
                d, v = self.scalar(e[2][1], e[2][0])
                p, q = unop_syntax(prec, e[1])
                return d, p + v + q
            d, v = self.scalar(prec, e[2][0])
            return d, self._unop(prec, e[1], v)
        if k == "tern":
            op = e[1]
            if op == "where":
                d1, v1 = self.scalar(e[2][1], e[2][0])      # condition keeps its precision
            else:
                d1, v1 = self.scalar(prec, e[2][0])
            d2, v2 = self.scalar(prec, e[3][0])
            d3, v3 = self.scalar(prec, e[4][0])
            return d1 + d2 + d3, self._ternop(prec, op, v1, v2, v3)
        raise ValueError("unknown scalar %r" % (k,))

    @staticmethod
    def _defs(defs) -> str:
        seen, out = set(), []
        for sid, doc in sorted(defs, key=lambda x: x[0]):
            if sid not in seen:
                seen.add(sid)
                out.append(doc)
        return "\n".join(out)

    @staticmethod
    def _block(defs: str, stmt: str) -> str:
        if not defs:
            return stmt
        return "{\n" + defs + "\n" + stmt + "\n}"

    # -- statements (c_syntax.ml:441-704)
    def stmt(self, s, in_loop=False) -> str:
        k = s[0]
        if k == "noop":
            return ""
        if k == "seq":
            return "\n".join(d for d in (self.stmt(x, in_loop) for x in s[1:]) if d)
        if k == "comment":
            return "/* " + s[1][1] + " */"
        if k == "for":
            i = s[1]
            return "for (%s %s = %d; %s <= %d; ++%s) {\n%s\n}" % (
                self.idx_t, i, int(s[2]), i, int(s[3]), i, self.stmt(s[4], True))
        if k == "zero_out":
            tid = int(s[1])
            t = self.tn[tid]
            first = tid not in self.zero_out_seen
            self.zero_out_seen.add(tid)
            if first and not in_loop and t["zero_init"] and t["mode"] == "local":
                return ""
            dims = t["dims"]
            # Low_level.loop_over_dims: size-1 axes are Fixed_idx 0, others get a loop
            idcs, nest = [], []
            for n, d in enumerate(dims):
                if d == 1:
                    idcs.append("0")
                else:
                    sym = "i_z%d_%d" % (tid, n)
                    idcs.append(sym)
                    nest.append((sym, d))
            body = ["set", str(tid), idcs, ["const", "0x0p+0"]]
            for sym, d in reversed(nest):
                body = ["for", sym, "0", str(d - 1), body]
            return self.stmt(body, in_loop)
        if k == "set":
            t = self.tn[int(s[1])]
            defs, val = self.scalar(t["prec"], s[3])
            a = "%s[%s] = %s;" % (t["ident"], self.offset(s[2], t["dims"]), val)
            return self._block(self._defs(defs), a)
        if k == "set_from_vec":
            # c_syntax.ml:548-592: one call, then `length` element stores; a Fixed_idx last
            # index is advanced per element, any other gets "+ i" on the computed offset
            t = self.tn[int(s[1])]
            length, op, (arg, arg_prec) = int(s[3]), s[4], s[5]
            assert op == "uint4x32_to_prec_uniform"
            defs, val = self.scalar(arg_prec, arg)
            vec_t = VEC_TYPE[(t["prec"], length)] if length > 1 else C_TYPE[t["prec"]]
            fn = "uint4x32_to_%s_uniform_vec(" % t["prec"]
            lines = ["%s vec_result = %s%s);" % (vec_t, fn, val)]
            idcs = list(s[2])
            for i in range(length):
                last = idcs[-1]
                if isinstance(last, str) and (last.isdigit() or (last[:1] == "-" and last[1:].isdigit())):
                    off = self.offset(idcs[:-1] + [str(int(last) + i)], t["dims"])
                else:
                    off = "%s + %d" % (self.offset(idcs, t["dims"]), i)
                lines.append("%s[%s] = %s;" % (t["ident"], off,
                                               "vec_result" if length == 1 else "vec_result.v[%d]" % i))
            return "{\n" + (self._defs(defs) + "\n" if defs else "") + "\n".join(lines) + "\n}"
        if k == "set_local":
            prec = self.tn[int(s[2])]["prec"]
            defs, val = self.scalar(prec, s[3])
            a = "%s = %s;" % (self.scope_name(s[1], s[2]), val)
            return self._block(self._defs(defs), a)
        if k == "declare_local":
            prec = self.tn[int(s[2])]["prec"]
            init = ""
            if int(s[3]):
                p, q = convert("int32", prec)
                init = " = " + p + "0" + q
            return "%s %s%s;" % (C_TYPE[prec], self.scope_name(s[1], s[2]), init)
        raise ValueError("unknown statement %r" % (k,))

    # -- the whole routine (c_syntax.ml:1021-1210)
    def params(self) -> List[Tuple[str, Tuple[str, object]]]:
        """Sorted (declaration, source) pairs; source is ('tn', id), ('static', sym) or
        ('merge', id)."""
        ps = []
        if self.merge is not None:
            ps.append(("const %s *merge_buffer" % C_TYPE[self.tn[self.merge]["prec"]],
                       ("merge", self.merge)))
        for sym, _ in self.static:
            ps.append(("const %s %s" % (self.idx_t, sym), ("static", sym)))
        for tid in self.order:
            t = self.tn[tid]
            if t["mode"] in ("ctx", "global"):
                ps.append(("%s *%s" % (C_TYPE[t["prec"]], t["ident"]), ("tn", tid)))
        # compare_string: bytewise order
        return sorted(ps, key=lambda p: p[0].encode())

    def function(self) -> str:
        self.zero_out_seen = set()
        ps = self.params()
        out = [" void %s(" % self.name]
        out.append(",\n".join("    " + d for d, _ in ps) + ") {")
        out.append("")
        out.append("  /* Local declarations and initialization. */")
        for tid in self.order:
            t = self.tn[tid]
            if t["mode"] == "local":
                n = math.prod(t["dims"]) if t["dims"] else 1
                out.append("  %s %s[%d]%s;" % (C_TYPE[t["prec"]], t["ident"], n,
                                               " = {0}" if t["zero_init"] else ""))
        out.append("")
        out.append("  /* Main logic. */")
        out.append(self.stmt(self.body))
        out.append("}")
        return "\n".join(out)

    def source(self) -> str:
        """A complete translation unit: the helper header + the routine."""
        return '#include "builtins_port.h"\n\n' + self.function() + "\n"


def emit(ir_text: str, large_models: bool = False) -> str:
    return Emitter(ir_text, large_models).source()
