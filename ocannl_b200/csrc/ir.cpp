// Parser for b200ir (see ir.hpp).  A small S-expression reader followed by a
// recursive descent over the constructors of `Low_level.t` / `scalar_t`.
#include "ir.hpp"

#include <cmath>
#include <cstdlib>
#include <cstring>

namespace b200 {

static const char* kPrecNames[] = {"byte", "uint16", "int32", "uint32", "int64", "uint64", "uint4x32",
                                   "half", "bfloat16", "fp8", "single", "double"};
static const int kPrecBytes[] = {1, 2, 4, 4, 8, 8, 16, 2, 2, 1, 4, 8};

Prec prec_of_string(const std::string& s) {
  for (int i = 0; i < 12; ++i)
    if (s == kPrecNames[i]) return (Prec)i;
  throw Error(-3, "b200ir: unknown precision '" + s + "'");
}
const char* prec_name(Prec p) { return kPrecNames[(int)p]; }
int prec_bytes(Prec p) { return kPrecBytes[(int)p]; }

namespace {

struct Sx {
  bool atom = false;
  bool quoted = false;
  std::string a;
  std::vector<Sx> l;
  const Sx& at(size_t i) const {
    if (atom || i >= l.size()) throw Error(-3, "b200ir: malformed list near '" + head() + "'");
    return l[i];
  }
  std::string head() const { return atom ? a : (l.empty() ? "()" : (l[0].atom ? l[0].a : "(")); }
  size_t size() const { return l.size(); }
};

struct Reader {
  const char* p;
  const char* e;
  int depth = 0;
  void ws() {
    while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  Sx read() {
    ws();
    if (p >= e) throw Error(-3, "b200ir: unexpected end of input");
    Sx x;
    if (*p == '(') {
      ++p;
      if (++depth > 4096) throw Error(-3, "b200ir: nesting too deep");
      for (;;) {
        ws();
        if (p >= e) throw Error(-3, "b200ir: unbalanced parentheses");
        if (*p == ')') {
          ++p;
          break;
        }
        x.l.push_back(read());
      }
      --depth;
      return x;
    }
    if (*p == ')') throw Error(-3, "b200ir: unexpected ')'");
    x.atom = true;
    if (*p == '"') {
      ++p;
      x.quoted = true;
      while (p < e && *p != '"') {
        if (*p == '\\' && p + 1 < e) ++p;
        x.a.push_back(*p++);
      }
      if (p >= e) throw Error(-3, "b200ir: unterminated string");
      ++p;
      return x;
    }
    while (p < e && *p != ' ' && *p != '\n' && *p != '\t' && *p != '\r' && *p != '(' && *p != ')') x.a.push_back(*p++);
    return x;
  }
};

int64_t to_int(const Sx& s) {
  if (!s.atom || s.a.empty()) throw Error(-3, "b200ir: integer expected");
  char* end = nullptr;
  long long v = strtoll(s.a.c_str(), &end, 10);
  if (*end) throw Error(-3, "b200ir: integer expected, got '" + s.a + "'");
  return v;
}

bool is_int_atom(const Sx& s) {
  if (!s.atom || s.a.empty()) return false;
  size_t i = (s.a[0] == '-') ? 1 : 0;
  if (i >= s.a.size()) return false;
  for (; i < s.a.size(); ++i)
    if (s.a[i] < '0' || s.a[i] > '9') return false;
  return true;
}

Index parse_index(const Sx& s) {
  Index ix;
  if (s.atom) {
    if (is_int_atom(s)) {
      ix.kind = Index::Fixed;
      ix.fixed = to_int(s);
    } else if (s.a == "sub_axis") {
      ix.kind = Index::SubAxis;
    } else {
      ix.kind = Index::Iter;
      ix.sym = s.a;
    }
    return ix;
  }
  if (s.head() != "affine") throw Error(-3, "b200ir: bad index form '" + s.head() + "'");
  ix.kind = Index::Affine;
  ix.fixed = to_int(s.at(1));
  for (size_t i = 2; i < s.size(); ++i) ix.terms.push_back({to_int(s.l[i].at(0)), s.l[i].at(1).a});
  return ix;
}

Indices parse_indices(const Sx& s) {
  if (s.atom) throw Error(-3, "b200ir: index list expected");
  Indices r;
  for (auto& x : s.l) r.push_back(parse_index(x));
  return r;
}

StmtP parse_stmt(const Sx& s);

Arg parse_arg(const Sx& s);

ScalarP parse_scalar(const Sx& s) {
  auto r = std::make_shared<Scalar>();
  const std::string h = s.head();
  if (h == "scope") {
    r->kind = Scalar::LocalScope;
    r->scope_id = (int)to_int(s.at(1));
    r->tn = (int)to_int(s.at(2));
    r->body = parse_stmt(s.at(3));
    r->idcs = parse_indices(s.at(4));
  } else if (h == "get_local") {
    r->kind = Scalar::GetLocal;
    r->scope_id = (int)to_int(s.at(1));
    r->tn = (int)to_int(s.at(2));
  } else if (h == "get" || h == "get_merge") {
    r->kind = h == "get" ? Scalar::Get : Scalar::GetMerge;
    r->tn = (int)to_int(s.at(1));
    r->idcs = parse_indices(s.at(2));
  } else if (h == "get_dyn") {
    r->kind = Scalar::GetDyn;
    r->tn = (int)to_int(s.at(1));
    r->idcs = parse_indices(s.at(2));
    r->dyn_axis = (int)to_int(s.at(3));
    r->args.push_back(parse_arg(s.at(4)));
  } else if (h == "tern") {
    r->kind = Scalar::Tern;
    r->op = s.at(1).a;
    for (int i = 2; i < 5; ++i) r->args.push_back(parse_arg(s.at(i)));
  } else if (h == "bin") {
    r->kind = Scalar::Bin;
    r->op = s.at(1).a;
    for (int i = 2; i < 4; ++i) r->args.push_back(parse_arg(s.at(i)));
  } else if (h == "un") {
    r->kind = Scalar::Un;
    r->op = s.at(1).a;
    r->args.push_back(parse_arg(s.at(2)));
  } else if (h == "const") {
    r->kind = Scalar::Const;
    const std::string& a = s.at(1).a;
    if (a == "inf")
      r->cval = INFINITY;
    else if (a == "-inf")
      r->cval = -INFINITY;
    else if (a == "nan")
      r->cval = NAN;
    else {
      char* end = nullptr;
      r->cval = strtod(a.c_str(), &end);  // accepts C99 hex floats
      if (end == a.c_str() || *end) throw Error(-3, "b200ir: bad constant '" + a + "'");
    }
  } else if (h == "const_bits") {
    r->kind = Scalar::ConstBits;
    r->bits = to_int(s.at(1));
  } else if (h == "idx") {
    r->kind = Scalar::EmbedIdx;
    r->idx = parse_index(s.at(1));
  } else {
    throw Error(-3, "b200ir: unknown scalar form '" + h + "'");
  }
  return r;
}

Arg parse_arg(const Sx& s) {
  Arg a;
  a.s = parse_scalar(s.at(0));
  a.prec = prec_of_string(s.at(1).a);
  return a;
}

StmtP parse_stmt(const Sx& s) {
  auto r = std::make_shared<Stmt>();
  const std::string h = s.head();
  if (h == "noop") {
    r->kind = Stmt::Noop;
  } else if (h == "comment") {
    r->kind = Stmt::Comment;
    r->text = s.at(1).a;
  } else if (h == "seq") {
    r->kind = Stmt::Seq;
    for (size_t i = 1; i < s.size(); ++i) r->items.push_back(parse_stmt(s.l[i]));
  } else if (h == "for") {
    r->kind = Stmt::For;
    r->index = s.at(1).a;
    r->from = to_int(s.at(2));
    r->to = to_int(s.at(3));
    r->body = parse_stmt(s.at(4));
  } else if (h == "zero_out") {
    r->kind = Stmt::ZeroOut;
    r->tn = (int)to_int(s.at(1));
  } else if (h == "set") {
    r->kind = Stmt::Set;
    r->tn = (int)to_int(s.at(1));
    r->idcs = parse_indices(s.at(2));
    r->value = parse_scalar(s.at(3));
  } else if (h == "set_from_vec") {
    r->kind = Stmt::Set;
    r->tn = (int)to_int(s.at(1));
    r->idcs = parse_indices(s.at(2));
    r->vec_len = (int)to_int(s.at(3));
    r->vec_op = s.at(4).a;
    if (r->vec_op != "uint4x32_to_prec_uniform" || r->vec_len < 1 || r->vec_len > 16)
      throw Error(-3, "b200ir: unsupported vector operation '" + r->vec_op + "'");
    Arg a = parse_arg(s.at(5));
    r->value = a.s;
    r->arg_prec = a.prec;
  } else if (h == "set_local") {
    r->kind = Stmt::SetLocal;
    r->scope_id = (int)to_int(s.at(1));
    r->tn = (int)to_int(s.at(2));
    r->value = parse_scalar(s.at(3));
  } else if (h == "declare_local") {
    r->kind = Stmt::DeclareLocal;
    r->scope_id = (int)to_int(s.at(1));
    r->tn = (int)to_int(s.at(2));
    r->needs_init = to_int(s.at(3)) != 0;
  } else {
    throw Error(-3, "b200ir: unknown statement form '" + h + "'");
  }
  return r;
}

}  // namespace

Program parse_program(const char* text, size_t len) {
  Reader rd{text, text + len};
  Sx root = rd.read();
  if (root.head() != "b200ir" || root.at(1).a != "1") throw Error(-3, "b200ir: expected (b200ir 1 ...)");
  Program pr;
  for (size_t i = 2; i < root.size(); ++i) {
    const Sx& sec = root.l[i];
    const std::string h = sec.head();
    if (h == "name") {
      pr.name = sec.at(1).a;
    } else if (h == "tnodes") {
      for (size_t k = 1; k < sec.size(); ++k) {
        const Sx& t = sec.l[k];
        Tnode tn;
        tn.id = (int)to_int(t.at(1));
        tn.ident = t.at(2).a;
        tn.prec = prec_of_string(t.at(3).a);
        for (auto& d : t.at(4).l) {
          int64_t v = to_int(d);
          if (v <= 0) throw Error(-3, "b200ir: non-positive dimension in node " + tn.ident);
          tn.dims.push_back(v);
        }
        const std::string& m = t.at(5).a;
        if (m == "virtual") tn.mode = Mode::Virtual;
        else if (m == "local") tn.mode = Mode::Local;
        else if (m == "ctx") tn.mode = Mode::Ctx;
        else if (m == "global") tn.mode = Mode::Global;
        else throw Error(-3, "b200ir: unknown memory mode '" + m + "'");
        for (size_t f = 6; f < t.size(); ++f) {
          if (t.l[f].a == "zero_init") tn.zero_init = true;
          else if (t.l[f].a == "read_only") tn.read_only = true;
        }
        if (pr.tn_index.count(tn.id)) throw Error(-3, "b200ir: duplicate node id " + std::to_string(tn.id));
        pr.tn_index[tn.id] = pr.tnodes.size();
        pr.tnodes.push_back(tn);
      }
    } else if (h == "static") {
      for (size_t k = 1; k < sec.size(); ++k) {
        StaticSym ss;
        ss.sym = sec.l[k].at(0).a;
        ss.range = sec.l[k].at(1).a == "none" ? -1 : to_int(sec.l[k].at(1));
        pr.statics.push_back(ss);
      }
    } else if (h == "merge") {
      pr.merge_node = sec.at(1).a == "none" ? -1 : (int)to_int(sec.at(1));
    } else if (h == "body") {
      pr.body = parse_stmt(sec.at(1));
    } else {
      throw Error(-3, "b200ir: unknown section '" + h + "'");
    }
  }
  if (pr.name.empty() || !pr.body) throw Error(-3, "b200ir: missing name or body");
  for (char c : pr.name)
    if (!(isalnum((unsigned char)c) || c == '_')) throw Error(-3, "b200ir: routine name must be a C identifier");
  return pr;
}

}  // namespace b200
