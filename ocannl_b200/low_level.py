"""Host-side mirror of arrayjit's for-loop IR and its wire format ("b200ir").

The classes restate the constructors of `Low_level.t` / `Low_level.scalar_t`
(arrayjit/lib/low_level.mli:22-68), `Indexing.axis_index`
(arrayjit/lib/indexing.ml:104-120) and the per-node facts of
`Low_level.traced_array` / `Low_level.optimized` (low_level.mli:104-166) that a
backend's `compile` receives.  `Routine.to_b200ir()` writes the S-expression
text that both the device library (`b200_compile`) and the CPU oracle parse.

Wire format (version 1):

    (b200ir 1 (name N)
      (tnodes (tn ID IDENT PREC (d0 d1 ..) MODE [zero_init] [read_only]) ..)
      (static (SYM RANGE|none) ..)
      (merge ID|none)
      (body STMT))
    STMT := (noop) | (comment "s") | (seq STMT ..) | (for SYM FROM TO STMT)
          | (zero_out ID) | (set ID (IDX ..) SC) | (set_local SID ID SC)
          | (declare_local SID ID 0|1)
    IDX  := INT | SYM | (affine OFFSET (COEFF SYM) ..) | sub_axis
    SC   := (scope SID ID STMT (IDX ..)) | (get_local SID ID) | (get ID (IDX ..))
          | (get_dyn ID (IDX ..) AXIS (SC PREC)) | (get_merge ID (IDX ..))
          | (tern OP (SC P) (SC P) (SC P)) | (bin OP (SC P) (SC P))
          | (un OP (SC P)) | (const HEXFLOAT) | (const_bits INT) | (idx IDX)

MODE is the memory class `C_syntax.compile_proc` derives per node
(arrayjit/lib/c_syntax.ml:1028-1043): `virtual`, `local`, `ctx` (in-context,
a kernel parameter) or `global` (materialised constant, also a parameter).
Loop bounds are inclusive, as in the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple, Union

PRECS = ("byte", "uint16", "int32", "uint32", "int64", "uint64", "uint4x32",
         "half", "bfloat16", "fp8", "single", "double")
PREC_BYTES = {"byte": 1, "uint16": 2, "int32": 4, "uint32": 4, "int64": 8, "uint64": 8,
              "uint4x32": 16, "half": 2, "bfloat16": 2, "fp8": 1, "single": 4, "double": 8}

BINOPS = ("arg1", "arg2", "add", "sub", "mul", "div", "pow", "relu_gate", "sat01_gate",
          "lt", "eq", "ne", "or", "and", "mod", "max", "min",
          "threefry4x32_crypto", "threefry4x32_light")
UNOPS = ("id", "relu", "sat01", "exp", "log", "exp2", "log2", "sin", "cos", "sqrt", "recip",
         "recip_sqrt", "neg", "trunc", "tanh", "not", "uint4x32_to_prec_uniform1")
# elements one uint4x32 yields per result precision (Ops.c_vec_typ_of_prec, arrayjit/lib/ops.ml:339-351)
VEC_LENGTH = {"single": 4, "double": 2, "int32": 4, "int64": 2, "byte": 16, "fp8": 16,
              "uint16": 8, "bfloat16": 8, "half": 8}
TERNOPS = ("where", "fma", "mul3")


# ---------------------------------------------------------------- tensor nodes
@dataclass(eq=False)
class Tnode:
    """Metadata of one tensor node (arrayjit/lib/tnode.ml): id, C identifier,
    precision, dims and memory class."""
    id: int
    ident: str
    prec: str
    dims: Tuple[int, ...]
    mode: str = "ctx"                 # virtual | local | ctx | global
    zero_init: bool = False           # traced_array.zero_initialized_by_code
    read_only: bool = False           # traced_array.read_only

    @property
    def num_elems(self) -> int:
        return int(math.prod(self.dims)) if self.dims else 1

    @property
    def size_in_bytes(self) -> int:
        return self.num_elems * PREC_BYTES[self.prec]

    def __getitem__(self, idcs) -> "Get":
        if not isinstance(idcs, tuple):
            idcs = (idcs,)
        return Get(self, tuple(idcs))


# ------------------------------------------------------------------- indices
@dataclass(frozen=True)
class Affine:
    """Σ coeff·symbol + offset (Indexing.Affine)."""
    terms: Tuple[Tuple[int, str], ...]
    offset: int = 0


Index = Union[int, str, Affine]       # Fixed_idx | Iterator | Affine ; "sub_axis" literal


def _idx_sexp(i: Index) -> str:
    if isinstance(i, Affine):
        return "(affine %d %s)" % (i.offset, " ".join("(%d %s)" % t for t in i.terms))
    return str(i)


def _idcs_sexp(idcs: Sequence[Index]) -> str:
    return "(" + " ".join(_idx_sexp(i) for i in idcs) + ")"


# ------------------------------------------------------------------- scalars
class Scalar:
    """Base of `scalar_t`; arithmetic operators build homogeneous Binops whose
    result precision follows `Low_level.scalar_precision` (promotion of the
    argument precisions by `Ops.promote_prec`)."""
    prec: str

    def _bin(self, op, other, rev=False):
        other = as_scalar(other, self.prec)
        a, b = (other, self) if rev else (self, other)
        return Binop(op, a, b)

    def __add__(self, o): return self._bin("add", o)
    def __radd__(self, o): return self._bin("add", o, True)
    def __sub__(self, o): return self._bin("sub", o)
    def __rsub__(self, o): return self._bin("sub", o, True)
    def __mul__(self, o): return self._bin("mul", o)
    def __rmul__(self, o): return self._bin("mul", o, True)
    def __truediv__(self, o): return self._bin("div", o)
    def __rtruediv__(self, o): return self._bin("div", o, True)
    def __pow__(self, o): return self._bin("pow", o)
    def __neg__(self): return Unop("neg", self)


_PROMO = {p: i for i, p in enumerate(
    ("byte", "uint16", "int32", "uint32", "int64", "uint64", "fp8", "half", "bfloat16",
     "single", "double", "uint4x32"))}


def promote(a: str, b: str) -> str:
    """Result precision of a homogeneous op on arguments of precisions a, b:
    `Ops.promote_prec` (arrayjit/lib/ops.ml:243-269) — a total order in which
    uint4x32 > double > single > bfloat16 > half > fp8 > the integer types."""
    return a if _PROMO[a] >= _PROMO[b] else b


def as_scalar(v, prec="single") -> Scalar:
    if isinstance(v, Scalar):
        return v
    return Const(float(v), prec)


@dataclass(eq=False)
class Const(Scalar):
    value: float
    prec: str = "single"

    def sexp(self):
        v = self.value
        if math.isinf(v):
            s = "inf" if v > 0 else "-inf"
        elif math.isnan(v):
            s = "nan"
        else:
            s = float(v).hex()
        return "(const %s)" % s


@dataclass(eq=False)
class ConstBits(Scalar):
    bits: int
    prec: str = "uint4x32"

    def sexp(self):
        return "(const_bits %d)" % self.bits


@dataclass(eq=False)
class EmbedIndex(Scalar):
    idx: Index
    prec: str = "uint32"

    def sexp(self):
        return "(idx %s)" % _idx_sexp(self.idx)


@dataclass(eq=False)
class Get(Scalar):
    tn: Tnode
    idcs: Tuple[Index, ...]

    @property
    def prec(self):
        return self.tn.prec

    def sexp(self):
        return "(get %d %s)" % (self.tn.id, _idcs_sexp(self.idcs))


@dataclass(eq=False)
class GetMerge(Scalar):
    tn: Tnode
    idcs: Tuple[Index, ...]

    @property
    def prec(self):
        return self.tn.prec

    def sexp(self):
        return "(get_merge %d %s)" % (self.tn.id, _idcs_sexp(self.idcs))


@dataclass(eq=False)
class GetDynamic(Scalar):
    """Guarded gather produced by `rewrite_one_hot_reductions`
    (arrayjit/lib/low_level.ml:2158-2329)."""
    tn: Tnode
    idcs: Tuple[Index, ...]
    dyn_axis: int
    dyn_value: Scalar

    @property
    def prec(self):
        return self.tn.prec

    def sexp(self):
        return "(get_dyn %d %s %d (%s %s))" % (self.tn.id, _idcs_sexp(self.idcs), self.dyn_axis,
                                               self.dyn_value.sexp(), self.dyn_value.prec)


@dataclass(eq=False)
class ScopeId:
    """`Low_level.scope_id`: a scalar local named v<scope_id>_<ident of tn>."""
    scope_id: int
    tn: Tnode


@dataclass(eq=False)
class LocalScope(Scalar):
    id: ScopeId
    body: "Stmt"
    orig_indices: Tuple[Index, ...] = ()

    @property
    def prec(self):
        return self.id.tn.prec

    def sexp(self):
        return "(scope %d %d %s %s)" % (self.id.scope_id, self.id.tn.id, self.body.sexp(),
                                        _idcs_sexp(self.orig_indices))


@dataclass(eq=False)
class GetLocal(Scalar):
    id: ScopeId

    @property
    def prec(self):
        return self.id.tn.prec

    def sexp(self):
        return "(get_local %d %d)" % (self.id.scope_id, self.id.tn.id)


def _arg(s: Scalar) -> str:
    return "(%s %s)" % (s.sexp(), s.prec)


@dataclass(eq=False)
class Binop(Scalar):
    op: str
    a: Scalar
    b: Scalar
    prec: str = ""

    def __post_init__(self):
        assert self.op in BINOPS, self.op
        if not self.prec:
            self.prec = promote(self.a.prec, self.b.prec)

    def sexp(self):
        return "(bin %s %s %s)" % (self.op, _arg(self.a), _arg(self.b))


@dataclass(eq=False)
class Unop(Scalar):
    op: str
    a: Scalar
    prec: str = ""

    def __post_init__(self):
        assert self.op in UNOPS, self.op
        if not self.prec:
            self.prec = self.a.prec

    def sexp(self):
        return "(un %s %s)" % (self.op, _arg(self.a))


@dataclass(eq=False)
class Ternop(Scalar):
    op: str
    a: Scalar
    b: Scalar
    c: Scalar
    prec: str = ""

    def __post_init__(self):
        assert self.op in TERNOPS, self.op
        if not self.prec:
            if self.op == "where":
                self.prec = promote(self.b.prec, self.c.prec)
            else:
                self.prec = promote(promote(self.a.prec, self.b.prec), self.c.prec)

    def sexp(self):
        return "(tern %s %s %s %s)" % (self.op, _arg(self.a), _arg(self.b), _arg(self.c))


def fma(a, b, c):
    return Ternop("fma", as_scalar(a), as_scalar(b), as_scalar(c))


def where(c, a, b):
    return Ternop("where", as_scalar(c), as_scalar(a), as_scalar(b))


def un(op, a):
    return Unop(op, as_scalar(a))


def binop(op, a, b):
    a = as_scalar(a)
    return Binop(op, a, as_scalar(b, a.prec))


# ---------------------------------------------------------------- statements
class Stmt:
    pass


@dataclass(eq=False)
class Noop(Stmt):
    def sexp(self):
        return "(noop)"


@dataclass(eq=False)
class Comment(Stmt):
    text: str

    def sexp(self):
        return '(comment "%s")' % self.text.replace("\\", "\\\\").replace('"', '\\"')


@dataclass(eq=False)
class Seq(Stmt):
    items: List[Stmt]

    def sexp(self):
        return "(seq %s)" % " ".join(s.sexp() for s in self.items)


@dataclass(eq=False)
class For(Stmt):
    index: str
    from_: int
    to_: int
    body: Stmt

    def sexp(self):
        return "(for %s %d %d %s)" % (self.index, self.from_, self.to_, self.body.sexp())


@dataclass(eq=False)
class ZeroOut(Stmt):
    tn: Tnode

    def sexp(self):
        return "(zero_out %d)" % self.tn.id


@dataclass(eq=False)
class Set(Stmt):
    tn: Tnode
    idcs: Tuple[Index, ...]
    llsc: Scalar

    def sexp(self):
        return "(set %d %s %s)" % (self.tn.id, _idcs_sexp(self.idcs), self.llsc.sexp())


@dataclass(eq=False)
class SetFromVec(Stmt):
    """`Set_from_vec {tn; idcs; length; vec_unop; arg}` (arrayjit/lib/low_level.mli:35-42): the
    vector operation's `length` results go to `length` consecutive elements starting at `idcs`.
    The only vector operation is `uint4x32_to_prec_uniform`, whose argument keeps its own
    (uint4x32) precision."""
    tn: Tnode
    idcs: Tuple[Index, ...]
    length: int
    arg: Scalar
    vec_unop: str = "uint4x32_to_prec_uniform"

    def sexp(self):
        return "(set_from_vec %d %s %d %s %s)" % (self.tn.id, _idcs_sexp(self.idcs), self.length,
                                                   self.vec_unop, _arg(self.arg))


@dataclass(eq=False)
class SetLocal(Stmt):
    id: ScopeId
    value: Scalar

    def sexp(self):
        return "(set_local %d %d %s)" % (self.id.scope_id, self.id.tn.id, self.value.sexp())


@dataclass(eq=False)
class DeclareLocal(Stmt):
    id: ScopeId
    needs_init: bool

    def sexp(self):
        return "(declare_local %d %d %d)" % (self.id.scope_id, self.id.tn.id, int(self.needs_init))


def loops(nest: Sequence[Tuple[str, int]], body: Stmt) -> Stmt:
    """for s0 = 0 to d0-1 { for s1 = 0 to d1-1 { ... body } }"""
    for sym, dim in reversed(list(nest)):
        body = For(sym, 0, dim - 1, body)
    return body


# ------------------------------------------------------------------ routine
@dataclass(eq=False)
class Routine:
    """What `Backend.compile ~name bindings lowered` receives
    (arrayjit/lib/backend_impl.ml:334-367): a name, the static index symbols
    (`Indexing.static_symbol`, indexing.ml:32-36) and `Low_level.optimized`."""
    name: str
    tnodes: List[Tnode] = field(default_factory=list)
    static: List[Tuple[str, Optional[int]]] = field(default_factory=list)
    merge_node: Optional[Tnode] = None
    body: Stmt = field(default_factory=Noop)
    _next_sym: int = 1
    _next_id: int = 1
    _next_scope: int = 1

    def tn(self, ident, prec, dims, mode="ctx", zero_init=False, read_only=False) -> Tnode:
        t = Tnode(self._next_id, ident, prec, tuple(int(d) for d in dims), mode, zero_init,
                  read_only)
        self._next_id += 1
        self.tnodes.append(t)
        return t

    def sym(self) -> str:
        s = "i%d" % self._next_sym
        self._next_sym += 1
        return s

    def syms(self, n):
        return [self.sym() for _ in range(n)]

    def static_sym(self, range_: Optional[int] = None) -> str:
        s = self.sym()
        self.static.append((s, range_))
        return s

    def scope(self, tn: Tnode) -> ScopeId:
        sid = ScopeId(self._next_scope, tn)
        self._next_scope += 1
        return sid

    def params(self) -> List[Tnode]:
        """Kernel parameters: the in-context / materialised nodes."""
        return [t for t in self.tnodes if t.mode in ("ctx", "global")]

    def to_b200ir(self) -> str:
        out = ["(b200ir 1 (name %s)" % self.name, " (tnodes"]
        for t in self.tnodes:
            flags = (" zero_init" if t.zero_init else "") + (" read_only" if t.read_only else "")
            out.append("  (tn %d %s %s (%s) %s%s)" % (
                t.id, t.ident, t.prec, " ".join(str(d) for d in t.dims), t.mode, flags))
        out.append(" )")
        out.append(" (static %s)" % " ".join(
            "(%s %s)" % (s, "none" if r is None else r) for s, r in self.static))
        out.append(" (merge %s)" % ("none" if self.merge_node is None else self.merge_node.id))
        out.append(" (body %s))" % self.body.sexp())
        return "\n".join(out) + "\n"
