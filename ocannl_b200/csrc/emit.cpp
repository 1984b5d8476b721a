// CUDA C emission of Low_level statements and scalars (see emit.hpp for the contract).
#include "emit.hpp"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>

namespace b200 {

namespace {
bool same_index(const Index& a, const Index& b) {
  return a.kind == b.kind && a.fixed == b.fixed && a.sym == b.sym && a.terms == b.terms;
}
bool same_indices(const Indices& a, const Indices& b) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i)
    if (!same_index(a[i], b[i])) return false;
  return true;
}
std::string pad(int n) { return std::string((size_t)n, ' '); }
bool lowp(Prec p) { return p == Prec::Bfloat16 || p == Prec::Half; }
// Inside expressions a bf16 / half value is a FLOAT that holds a value representable in that
// format ("rounded float"): one rounding step per operation, no unpack / repack between
// operations.  Storage stays 16 bits; loads widen, stores take the (already exact) 16 bits.
const char* round_fn(Prec p) { return p == Prec::Bfloat16 ? "b200_rbf(" : "b200_rhf("; }
}  // namespace

const char* Emitter::rtype(Prec p) { return lowp(p) ? "float" : ctype(p); }
std::string Emitter::load_wrap(Prec p, const std::string& e) {
  if (p == Prec::Bfloat16) return "b200_bf2f(" + e + ")";
  if (p == Prec::Half) return "b200_h2f(" + e + ")";
  return e;
}
std::string Emitter::store_wrap(Prec p, const std::string& e) {
  if (p == Prec::Bfloat16) return "b200_bfbits(" + e + ")";
  if (p == Prec::Half) return "b200_f2h(" + e + ")";
  return e;
}
std::string Emitter::storage_zero(Prec p) {
  if (lowp(p)) return "((unsigned short)0)";
  return constant(0.0, p);
}

const char* Emitter::ctype(Prec p) {
  switch (p) {
    case Prec::Byte: return "unsigned char";
    case Prec::Uint16: return "unsigned short";
    case Prec::Int32: return "int";
    case Prec::Uint32: return "unsigned int";
    case Prec::Int64: return "long long";
    case Prec::Uint64: return "unsigned long long";
    case Prec::Half: return "unsigned short";
    case Prec::Bfloat16: return "unsigned short";
    case Prec::Single: return "float";
    case Prec::Double: return "double";
    case Prec::Uint4x32: return "b200_u4x32";
    case Prec::Fp8: return "unsigned char";   // the 8 bits; arithmetic widens them (see convert / binop)
  }
  throw Error(-3, "b200ir: unknown precision");
}

// Ops.c_convert_precision (arrayjit/lib/ops.ml:798-863) for the device spellings.
std::pair<std::string, std::string> Emitter::convert(Prec from, Prec to) {
  if (from == to) return {"", ""};
  if (from == Prec::Fp8 || to == Prec::Fp8) {
    // through single precision, as Ops.c_convert_precision spells it (arrayjit/lib/ops.ml:798-863);
    // an 8-bit value is its code inside expressions
    if (to == Prec::Uint4x32) return {"b200_word_to_u4x32((b200_u32)(", "))"};
    if (from == Prec::Uint4x32) throw Error(-4, "unsupported uint4x32 conversion");
    if (to == Prec::Fp8) {
      // (rounded floats of 16-bit precisions are floats already)
      if (from == Prec::Single || lowp(from)) return {"b200_f2fp8(", ")"};
      return {"b200_f2fp8((float)(", "))"};
    }
    auto out = convert(Prec::Single, to);
    return {out.first + "b200_fp82f(", ")" + out.second};
  }
  if (from == Prec::Uint4x32 || to == Prec::Uint4x32) {
    // arrayjit/lib/builtins.c:531-606
    if (to == Prec::Uint4x32) {
      if (from == Prec::Uint32 || from == Prec::Int32) return {"b200_u32_widen((b200_u32)(", "))"};
      if (from == Prec::Uint64 || from == Prec::Int64) return {"b200_u64_to_u4x32((b200_u64)(", "))"};
      if (from == Prec::Double) return {"b200_f64_to_u4x32(", ")"};
      if (from == Prec::Single) return {"b200_f32_to_u4x32(", ")"};
      if (from == Prec::Byte || from == Prec::Uint16) return {"b200_word_to_u4x32((b200_u32)(", "))"};
      if (from == Prec::Bfloat16) return {"b200_word_to_u4x32((b200_u32)b200_bfbits(", "))"};
      if (from == Prec::Half) return {"b200_word_to_u4x32((b200_u32)b200_f2h(", "))"};
    }
    throw Error(-4, "unsupported uint4x32 conversion");
  }
  auto is_plain_int = [](Prec p) {
    return p == Prec::Byte || p == Prec::Uint16 || p == Prec::Int32 || p == Prec::Uint32 || p == Prec::Int64 ||
           p == Prec::Uint64;
  };
  if (lowp(from)) {
    if (to == Prec::Single) return {"", ""};                       // already a float
    if (to == Prec::Double) return {"(double)(", ")"};
    if (lowp(to)) return {round_fn(to), ")"};                      // bf16 <-> half
    return {std::string("(") + ctype(to) + ")(", ")"};
  }
  if (lowp(to)) {
    if (from == Prec::Single) return {round_fn(to), ")"};
    return {std::string(round_fn(to)) + "(float)(", "))"};        // double and the integer types
  }
  (void)is_plain_int;
  return {std::string("(") + ctype(to) + ")(", ")"};
}

std::string Emitter::index(const Index& ix) {
  switch (ix.kind) {
    case Index::Fixed: return std::to_string(ix.fixed);
    case Index::Iter: return (pair_hi && ix.sym == pair_sym) ? "(" + ix.sym + "+1u)" : ix.sym;
    case Index::SubAxis: return "";
    case Index::Affine: {
      std::string r;
      for (auto& t : ix.terms) {
        if (!r.empty()) r += "+";
        const std::string sym = (pair_hi && t.second == pair_sym) ? "(" + t.second + "+1u)" : t.second;
        r += t.first == 1 ? sym : std::to_string(t.first) + "*" + sym;
      }
      if (ix.fixed > 0) r += (r.empty() ? "" : "+") + std::to_string(ix.fixed);
      else if (ix.fixed < 0) r += (r.empty() ? "" : "+") + std::string("-") + std::to_string(-ix.fixed);
      return r.empty() ? "0" : r;
    }
  }
  return "0";
}

// C_syntax.pp_array_offset (arrayjit/lib/c_syntax.ml:367-379)
std::string Emitter::offset(const Indices& idcs, const std::vector<int64_t>& dims, int dyn_axis,
                            const std::string& dyn_doc) {
  if (idcs.empty()) return "0";
  if (idcs.size() != dims.size()) throw Error(-3, "b200ir: index count does not match the node's rank");
  auto ax = [&](size_t k) { return (int)k == dyn_axis ? dyn_doc : index(idcs[k]); };
  std::string doc = ax(0);
  for (size_t k = 1; k < idcs.size(); ++k) {
    std::string d = ax(k);
    if (doc.empty()) doc = d;
    else if (d.empty()) doc = "(" + doc + ") * " + std::to_string(dims[k]);
    else doc = "(" + doc + ") * " + std::to_string(dims[k]) + " + " + d;
  }
  return doc;
}

std::string Emitter::scope_name(int scope_id, int tn) const {
  return "v" + std::to_string(scope_id) + "_" + P.tn(tn).ident;
}
std::string Emitter::node_name(int tn) const { return P.tn(tn).ident; }

// the value of `c` rounded to a 16-bit format, as a float
static float round_lowp(double c, Prec prec) {
  const float f = (float)c;
  if (prec == Prec::Bfloat16) {
    unsigned int u;
    float rounded;
    memcpy(&u, &f, 4);
    if (std::isnan(f)) return f;
    u += 0x7FFFu + ((u >> 16) & 1u);  // arrayjit/lib/builtins.c:620-627
    u &= 0xFFFF0000u;
    memcpy(&rounded, &u, 4);
    return rounded;
  }
  return (float)(_Float16)f;
}
// ... and its 16 storage bits
static unsigned int lowp_bits(double c, Prec prec) {
  const float r = round_lowp(c, prec);
  if (prec == Prec::Bfloat16) {
    unsigned int u;
    memcpy(&u, &r, 4);
    return std::isnan(r) ? 0x7FFFu : (u >> 16);
  }
  const _Float16 h = (_Float16)r;
  unsigned short b;
  memcpy(&b, &h, 2);
  return b;
}

// the reference's float -> 8-bit float narrowing (arrayjit/lib/builtins.c:688-742), for constants
static unsigned int fp8_bits(float f) {
  if (f == 0.0f) return 0;
  const unsigned int sign = f < 0 ? 1u : 0u;
  f = std::fabs(f);
  if (std::isinf(f)) return (sign << 7) | 0x7Cu;
  if (std::isnan(f)) return (sign << 7) | 0x7Fu;
  int ex;
  const float m = std::frexp(f, &ex);
  const int e = ex + 14;
  if (e < 0) return sign << 7;
  if (e > 30) return (sign << 7) | 0x7Cu;
  unsigned int bits;
  if (e == 0) {
    bits = (unsigned int)(f * std::ldexp(1.0f, 14) * 4.0f + 0.5f);
    return (sign << 7) | (bits > 3u ? 3u : bits);
  }
  bits = (unsigned int)((m - 0.5f) * 4.0f + 0.5f);
  return (sign << 7) | (((unsigned int)e & 0x1Fu) << 2) | (bits > 3u ? 3u : bits);
}

std::string Emitter::constant(double c, Prec prec) {
  char buf[64];
  if (prec == Prec::Fp8) {
    snprintf(buf, sizeof buf, "((unsigned char)0x%02xu)", fp8_bits((float)c));
    return buf;
  }
  if (prec == Prec::Uint4x32) {
    snprintf(buf, sizeof buf, "%a", c);
    return std::string("b200_f64_to_u4x32(") + buf + ")";
  }
  if (prec == Prec::Single || lowp(prec)) {
    std::string lit;
    if (std::isinf(c)) lit = c > 0 ? "B200_INF" : "(-B200_INF)";
    else if (std::isnan(c)) lit = "B200_NAN";
    else {
      snprintf(buf, sizeof buf, "%a", (double)(float)c);
      lit = std::string(buf) + "f";
      if (c < 0) lit = "(" + lit + ")";
    }
    if (prec == Prec::Single) return lit;
    // 16-bit constants are rounded here, once, instead of per element on the device
    const float rounded = round_lowp(c, prec);
    if (std::isinf(rounded)) return rounded > 0 ? "B200_INF" : "(-B200_INF)";
    if (std::isnan(rounded)) return "B200_NAN";
    snprintf(buf, sizeof buf, "%a", (double)rounded);
    lit = std::string(buf) + "f";
    if (rounded < 0) lit = "(" + lit + ")";
    return lit;
  }
  if (prec == Prec::Double) {
    if (std::isinf(c)) return c > 0 ? "((double)B200_INF)" : "(-(double)B200_INF)";
    if (std::isnan(c)) return "((double)B200_NAN)";
    snprintf(buf, sizeof buf, "%a", c);
    return c < 0 ? "(" + std::string(buf) + ")" : std::string(buf);
  }
  snprintf(buf, sizeof buf, "%a", c);
  return std::string("(") + ctype(prec) + ")(" + buf + ")";
}

// Ops.binop_c_syntax / unop_c_syntax / ternop_c_syntax with device literals.
static std::string binop_plain(Prec prec, const std::string& op, const std::string& a, const std::string& b) {
  const bool dbl = prec == Prec::Double;
  const bool integ = is_int_prec(prec);
  const std::string zero = integ ? "0" : (dbl ? "0.0" : "0.0f");
  const std::string T = Emitter::ctype(prec);
  if (op == "add") return "(" + a + " + " + b + ")";
  if (op == "sub") return "(" + a + " - " + b + ")";
  if (op == "mul") return "(" + a + " * " + b + ")";
  if (op == "div") return (!integ && !dbl) ? "b200_fdiv(" + a + ", " + b + ")" : "(" + a + " / " + b + ")";
  if (op == "pow") {
    if (integ) throw Error(-4, "pow is not defined for integer precisions");
    return (dbl ? "pow(" : "powf(") + a + ", " + b + ")";
  }
  if (op == "relu_gate") return "(" + a + " > " + zero + " ? " + b + " : " + zero + ")";
  if (op == "sat01_gate") {
    if (integ) return "(abs(" + a + ") > 0 ? 0 : (" + b + "))";
    return (dbl ? "(fabs(floor(" : "(fabsf(floorf(") + a + ")) > " + zero + " ? " + zero + " : (" + b + "))";
  }
  if (op == "max" || op == "min") {
    if (integ) return "(" + T + ")f" + op + "((double)(" + a + "), (double)(" + b + "))";
    return std::string("f") + op + (dbl ? "(" : "f(") + a + ", " + b + ")";
  }
  if (op == "mod") return "(" + a + " % " + b + ")";
  const char* sym = op == "lt" ? "<" : op == "eq" ? "==" : op == "ne" ? "!=" : op == "or" ? "||" : op == "and" ? "&&" : nullptr;
  if (sym) return "((" + T + ")(" + a + " " + sym + " " + b + "))";
  throw Error(-4, "unsupported binary operation '" + op + "'");
}

static std::string unop_plain(Prec prec, const std::string& op, const std::string& v) {
  const bool dbl = prec == Prec::Double;
  const bool integ = is_int_prec(prec);
  const std::string zero = integ ? "0" : (dbl ? "0.0" : "0.0f");
  const std::string one = integ ? "1" : (dbl ? "1.0" : "1.0f");
  const std::string T = Emitter::ctype(prec);
  auto fn = [&](const char* name) {
    if (integ) return "(" + T + ")" + name + "((double)(" + v + "))";
    return std::string(name) + (dbl ? "(" : "f(") + v + ")";
  };
  if (op == "id") return v;
  if (op == "relu") {
    if (integ) return "(" + T + ")fmax(0.0, (double)(" + v + "))";
    return std::string(dbl ? "fmax(" : "fmaxf(") + zero + ", " + v + ")";
  }
  if (op == "sat01") {
    if (integ) return "(" + T + ")fmax(0.0, fmin(1.0, (double)(" + v + ")))";
    return std::string(dbl ? "fmax(" : "fmaxf(") + zero + ", " + (dbl ? "fmin(" : "fminf(") + one + ", " + v + "))";
  }
  if (op == "exp" || op == "log" || op == "exp2" || op == "log2" || op == "sin" || op == "cos" || op == "sqrt")
    return fn(op.c_str());
  if (integ && (op == "recip" || op == "recip_sqrt" || op == "tanh"))
    throw Error(-4, "operation '" + op + "' is not defined for integer precisions");
  if (op == "recip") return "(" + one + " / (" + v + "))";
  if (op == "recip_sqrt") return "(" + one + " / " + (dbl ? "sqrt(" : "sqrtf(") + v + "))";
  if (op == "neg") return "(-(" + v + "))";
  if (op == "trunc") return dbl ? "trunc(" + v + ")" : "truncf(" + v + ")";
  // the reference spells tanh `tanhf(` for every floating precision, double included
  // (arrayjit/lib/ops.ml:765-769): a double argument is narrowed, the float result widened
  if (op == "tanh") return dbl ? "(double)tanhf((float)(" + v + "))" : "tanhf(" + v + ")";
  if (op == "not") return "(" + v + " == " + zero + " ? " + one + " : " + zero + ")";
  throw Error(-4, "unsupported unary operation '" + op + "'");
}

static std::string ternop_plain(Prec prec, const std::string& op, const std::string& a, const std::string& b,
                                const std::string& c) {
  const bool dbl = prec == Prec::Double;
  const bool integ = is_int_prec(prec);
  if (op == "where") return "((" + a + ") != 0 ? (" + b + ") : (" + c + "))";
  if (op == "fma") {
    if (integ) return "((" + a + ") * (" + b + ") + (" + c + "))";
    return std::string(dbl ? "fma(" : "fmaf(") + a + ", " + b + ", " + c + ")";
  }
  if (op == "mul3") return "((" + a + ") * (" + b + ") * (" + c + "))";
  throw Error(-4, "unsupported ternary operation '" + op + "'");
}

// Operations whose result, for arguments that are already values of a 16-bit format, is again
// such a value (one of the arguments, its sign flip or truncation, or 0 / 1): no rounding step.
static bool selects_exactly(const std::string& op) {
  static const std::set<std::string> k = {"relu_gate", "sat01_gate", "max", "min", "lt", "eq", "ne", "or", "and",
                                          "relu", "sat01", "neg", "trunc", "not", "where"};
  return k.count(op) != 0;
}

std::string Emitter::binop(Prec prec, const std::string& op, const std::string& a, const std::string& b) {
  if (op == "threefry4x32_crypto" || op == "threefry4x32_light") {
    if (prec != Prec::Uint4x32) throw Error(-4, "threefry4x32 outside a uint4x32 context");
    return (op == "threefry4x32_crypto" ? "b200_threefry_crypto(" : "b200_threefry_light(") + a + ", " + b + ")";
  }
  // 8-bit floats: widen, operate in float, narrow -- every time (arrayjit/lib/cc_backend.ml:169-322)
  if (prec == Prec::Fp8) return "b200_f2fp8(" + binop_plain(Prec::Single, op, "b200_fp82f(" + a + ")", "b200_fp82f(" + b + ")") + ")";
  if (lowp(prec) && selects_exactly(op)) return binop_plain(Prec::Single, op, a, b);
  if (op == "div" && (lowp(prec) || prec == Prec::Single)) {
    {
      // a power of two: the quotient is the product with its reciprocal, bit for bit
      int e2 = 0;
      char tail = 0;
      if (sscanf(b.c_str(), "0x1p%d%c", &e2, &tail) == 2 && tail == 'f' && b.size() <= 10 && e2 > -100 && e2 < 100) {
        char r[32];
        snprintf(r, sizeof r, "0x1p%+df", -e2);
        const std::string q = "(" + a + " * " + r + ")";
        return lowp(prec) ? std::string(round_fn(prec)) + q + ")" : q;
      }
    }
    if (divisor_probe) divisor_probe->push_back(b);
    // a divisor that the caller prepared once for many numerators (see b200_divisor in numerics.cuh)
    auto it = divisor_vars.find(b);
    if (it != divisor_vars.end()) {
      const std::string q = "b200_div_by(" + a + ", " + it->second + ")";
      return lowp(prec) ? std::string(round_fn(prec)) + q + ")" : q;
    }
  }
  if (lowp(prec)) return std::string(round_fn(prec)) + binop_plain(Prec::Single, op, a, b) + ")";
  return binop_plain(prec, op, a, b);
}
std::string Emitter::unop(Prec prec, const std::string& op, const std::string& a) {
  if (prec == Prec::Fp8) {
    if (op == "id") return a;
    return "b200_f2fp8(" + unop_plain(Prec::Single, op, "b200_fp82f(" + a + ")") + ")";
  }
  if (lowp(prec)) {
    // a 16-bit result keeps 8 (bf16) or 11 (half) significant bits: the hardware
    // approximations of tanh / exp / log (relative error below 2^-10) round to the same value
    // as the libm functions except for rare one-unit differences in the last kept bit
    if (op == "id") return a;
    if (selects_exactly(op)) return unop_plain(Prec::Single, op, a);
    if (op == "tanh") return std::string(round_fn(prec)) + "b200_tanh_fast(" + a + "))";
    if (op == "exp") return std::string(round_fn(prec)) + "__expf(" + a + "))";
    if (op == "log") return std::string(round_fn(prec)) + "__logf(" + a + "))";
    return std::string(round_fn(prec)) + unop_plain(Prec::Single, op, a) + ")";
  }
  return unop_plain(prec, op, a);
}
std::string Emitter::ternop(Prec prec, const std::string& op, const std::string& a, const std::string& b,
                            const std::string& c) {
  if (prec == Prec::Fp8)
    return "b200_f2fp8(" + ternop_plain(Prec::Single, op, "b200_fp82f(" + a + ")", "b200_fp82f(" + b + ")", "b200_fp82f(" + c + ")") + ")";
  if (lowp(prec) && selects_exactly(op)) return ternop_plain(Prec::Single, op, a, b, c);
  if (lowp(prec)) return std::string(round_fn(prec)) + ternop_plain(Prec::Single, op, a, b, c) + ")";
  return ternop_plain(prec, op, a, b, c);
}

// Low_level.reads_scope_before_set (arrayjit/lib/low_level.ml:1998-2037)
bool Emitter::reads_scope_before_set(int scope_id, int tn, const Stmt& body) {
  struct W {
    int sid, tn;
    bool sc_reads(const Scalar& e) const {
      switch (e.kind) {
        case Scalar::GetLocal: return e.scope_id == sid && e.tn == tn;
        case Scalar::LocalScope: return st_reads(*e.body);
        case Scalar::GetDyn: return sc_reads(*e.args[0].s);
        case Scalar::Tern:
        case Scalar::Bin:
        case Scalar::Un:
          for (auto& a : e.args)
            if (sc_reads(*a.s)) return true;
          return false;
        default: return false;
      }
    }
    bool st_reads(const Stmt& s) const {
      switch (s.kind) {
        case Stmt::Seq:
          for (auto& x : s.items)
            if (st_reads(*x)) return true;
          return false;
        case Stmt::For: return st_reads(*s.body);
        case Stmt::Set:
        case Stmt::SetLocal: return sc_reads(*s.value);
        default: return false;
      }
    }
    // 0 neither, 1 read, 2 written
    int scan(const Stmt& s) const {
      switch (s.kind) {
        case Stmt::Set: return sc_reads(*s.value) ? 1 : 0;
        case Stmt::SetLocal:
          if (sc_reads(*s.value)) return 1;
          return (s.scope_id == sid && s.tn == tn) ? 2 : 0;
        case Stmt::Seq:
          for (auto& x : s.items) {
            int r = scan(*x);
            if (r) return r;
          }
          return 0;
        case Stmt::For: {
          int r = scan(*s.body);
          if (r == 2) return s.from <= s.to ? 2 : 0;
          return r;
        }
        default: return 0;
      }
    }
  } w{scope_id, tn};
  return w.scan(body) != 2;
}

Emitter::Res Emitter::scalar(Prec prec, const Scalar& e) {
  Res r;
  switch (e.kind) {
    case Scalar::LocalScope: {
      Prec sp = P.tn(e.tn).prec;
      auto cv = convert(sp, prec);
      auto sub = scope_subst.find(e.scope_id);
      if (sub != scope_subst.end()) {
        r.expr = cv.first + sub->second + cv.second;
        return r;
      }
      std::string init;
      if (reads_scope_before_set(e.scope_id, e.tn, *e.body)) init = " = " + constant(0.0, sp);
      std::string def = std::string(rtype(sp)) + " " + scope_name(e.scope_id, e.tn) + init + ";\n" + stmt(*e.body, 0);
      r.defs.push_back({e.scope_id, def});
      r.expr = cv.first + scope_name(e.scope_id, e.tn) + cv.second;
      return r;
    }
    case Scalar::GetLocal: {
      auto cv = convert(P.tn(e.tn).prec, prec);
      auto sub = scope_subst.find(e.scope_id);
      r.expr = cv.first + (sub != scope_subst.end() ? sub->second : scope_name(e.scope_id, e.tn)) + cv.second;
      return r;
    }
    case Scalar::Get:
    case Scalar::GetMerge: {
      const Tnode& t = P.tn(e.tn);
      auto cv = convert(t.prec, prec);
      if (e.kind == Scalar::Get) {
        auto f = forwarded.find(e.tn);
        if (f != forwarded.end() && same_indices(f->second.first, e.idcs)) {
          r.expr = cv.first + f->second.second + cv.second;
          return r;
        }
        for (auto& rf : row_forwards) {
          if (rf.tn != e.tn || rf.idcs.size() != e.idcs.size()) continue;
          bool ok = true;
          std::string sub;
          for (size_t a = 0; ok && a < e.idcs.size(); ++a) {
            Index x = e.idcs[a];
            if ((int)a == rf.n_axis) {
              if (x.kind == Index::Iter) sub = rf.fixed_index.empty() ? "[" + x.sym + rf.index_shift + "]" : "[" + rf.fixed_index + "]";
              else if (x.kind == Index::Fixed && rf.index_shift.empty()) sub = "[" + std::to_string(x.fixed) + "]";
              else ok = false;
            } else {
              if (x.kind == Index::Iter) {
                auto it = row_ren.find(x.sym);
                if (it != row_ren.end()) x.sym = it->second;
              }
              ok = same_index(x, rf.idcs[a]);
            }
          }
          if (ok) {
            r.expr = cv.first + rf.name + sub + cv.second;
            return r;
          }
        }
        if (t.mode == Mode::Virtual) throw Error(-3, "b200ir: read of virtual node '" + t.ident + "'");
        used_nodes.insert(e.tn);
        for (auto& lt : load_tiles)
          if (lt.tn == e.tn && same_indices(lt.idcs, e.idcs)) {
            r.expr = cv.first + load_wrap(t.prec, lt.expr) + cv.second;   // tiles hold storage bits
            return r;
          }
      } else {
        uses_merge = true;
      }
      std::string name = e.kind == Scalar::GetMerge ? "merge_buffer" : t.ident;
      if (e.kind == Scalar::Get) {
        auto al = node_alias.find(e.tn);
        if (al != node_alias.end()) name = al->second;
      }
      ++direct_reads;
      r.expr = cv.first + load_wrap(t.prec, name + "[" + offset(e.idcs, t.dims) + "]") + cv.second;
      return r;
    }
    case Scalar::GetDyn: {
      const Tnode& t = P.tn(e.tn);
      auto cv = convert(t.prec, prec);
      Res d = scalar(e.args[0].prec, *e.args[0].s);
      used_nodes.insert(e.tn);
      ++direct_reads;
      std::string dyn = std::string("((") + (large_models ? "unsigned long long" : "unsigned int") + ")(" + d.expr + "))";
      r.defs = d.defs;
      r.expr = cv.first + load_wrap(t.prec, t.ident + "[" + offset(e.idcs, t.dims, e.dyn_axis, dyn) + "]") + cv.second;
      return r;
    }
    case Scalar::Const: r.expr = constant(e.cval, prec); return r;
    case Scalar::ConstBits: {
      auto cv = convert(Prec::Int64, prec);
      r.expr = cv.first + std::to_string(e.bits) + "LL" + cv.second;
      return r;
    }
    case Scalar::EmbedIdx: {
      auto cv = convert(large_models ? Prec::Uint64 : Prec::Uint32, prec);
      std::string d = index(e.idx);
      r.expr = cv.first + (d.empty() ? "0" : d) + cv.second;
      return r;
    }
    case Scalar::Bin: {
      if (e.op == "arg1") return scalar(prec, *e.args[0].s);
      if (e.op == "arg2") return scalar(prec, *e.args[1].s);
      if (e.op == "pow" && e.args[1].s->kind == Scalar::Const && !is_int_prec(prec) &&
          (e.args[1].s->cval == 2.0 || e.args[1].s->cval == 3.0)) {
        // x ** 2 and x ** 3 by multiplication (within 2 ulp of powf, far cheaper in an epilogue)
        Res a = scalar(prec, *e.args[0].s);
        r.defs = a.defs;
        const std::string fn = e.args[1].s->cval == 2.0 ? "b200_pow2(" : "b200_pow3(";
        if (lowp(prec)) r.expr = std::string(round_fn(prec)) + fn + a.expr + "))";
        else r.expr = fn + a.expr + ")";
        return r;
      }
      Res a = scalar(prec, *e.args[0].s), b = scalar(prec, *e.args[1].s);
      r.defs = a.defs;
      r.defs.insert(r.defs.end(), b.defs.begin(), b.defs.end());
      r.expr = binop(prec, e.op, a.expr, b.expr);
      return r;
    }
    case Scalar::Un: {
      if (e.op == "uint4x32_to_prec_uniform1") {
        // not homogeneous: the argument keeps its own (uint4x32) precision
        Res a = scalar(e.args[0].prec, *e.args[0].s);
        r.defs = a.defs;
        if (e.args[0].prec != Prec::Uint4x32) throw Error(-4, "uint4x32_to_prec_uniform1 of a non-uint4x32 argument");
        switch (prec) {
          case Prec::Single: r.expr = "b200_uniform_single(" + a.expr + ", 0)"; break;
          case Prec::Double: r.expr = "b200_uniform_double(" + a.expr + ", 0)"; break;
          case Prec::Int32: r.expr = "b200_uniform_int32(" + a.expr + ", 0)"; break;
          case Prec::Uint32: r.expr = "(b200_u32)b200_uniform_int32(" + a.expr + ", 0)"; break;
          case Prec::Int64: r.expr = "b200_uniform_int64(" + a.expr + ", 0)"; break;
          case Prec::Uint64: r.expr = "(b200_u64)b200_uniform_int64(" + a.expr + ", 0)"; break;
          case Prec::Bfloat16: r.expr = load_wrap(prec, "b200_uniform1_bfloat16(" + a.expr + ")"); break;
          case Prec::Half: r.expr = load_wrap(prec, "b200_uniform_half(" + a.expr + ", 0)"); break;
          case Prec::Fp8:
          case Prec::Byte: r.expr = "((unsigned char)((" + a.expr + ").v[0] & 0xFFu))"; break;   // builtins.c:415-418
          default: throw Error(-4, "uint4x32_to_prec_uniform1 into an unsupported precision");
        }
        return r;
      }
      Res a = scalar(prec, *e.args[0].s);
      r.defs = a.defs;
      r.expr = unop(prec, e.op, a.expr);
      return r;
    }
    case Scalar::Tern: {
      const bool is_where = e.op == "where";
      Res a = scalar(is_where ? e.args[0].prec : prec, *e.args[0].s);
      Res b = scalar(prec, *e.args[1].s), c = scalar(prec, *e.args[2].s);
      r.defs = a.defs;
      r.defs.insert(r.defs.end(), b.defs.begin(), b.defs.end());
      r.defs.insert(r.defs.end(), c.defs.begin(), c.defs.end());
      if (is_where) {
        // the condition keeps its own precision: compare it there, select in `prec`
        std::string cond = a.expr;
        if (e.args[0].prec == Prec::Fp8) cond = "b200_fp82f(" + cond + ")";   // a code is compared as the number it stands for
        if (prec == Prec::Fp8)   // the selected value is widened and narrowed like any other result
          r.expr = "b200_f2fp8((" + cond + ") != 0 ? b200_fp82f(" + b.expr + ") : b200_fp82f(" + c.expr + "))";
        else
          r.expr = "((" + cond + ") != 0 ? (" + b.expr + ") : (" + c.expr + "))";
      } else {
        r.expr = ternop(prec, e.op, a.expr, b.expr, c.expr);
      }
      return r;
    }
  }
  throw Error(-3, "b200ir: unknown scalar");
}

static std::string emit_defs(std::vector<std::pair<int, std::string>> defs, int indent) {
  std::stable_sort(defs.begin(), defs.end(), [](auto& a, auto& b) { return a.first < b.first; });
  std::string out;
  int last = -1;
  bool first = true;
  for (auto& d : defs) {
    if (!first && d.first == last) continue;
    first = false;
    last = d.first;
    // re-indent the definition text
    size_t pos = 0;
    while (pos < d.second.size()) {
      size_t nl = d.second.find('\n', pos);
      std::string line = d.second.substr(pos, nl == std::string::npos ? std::string::npos : nl - pos);
      if (!line.empty()) out += pad(indent) + line + "\n";
      if (nl == std::string::npos) break;
      pos = nl + 1;
    }
  }
  return out;
}

std::string Emitter::stmt(const Stmt& s, int ind) {
  switch (s.kind) {
    case Stmt::Noop: return "";
    case Stmt::Comment: {
      std::string t = s.text;
      for (size_t p = 0; (p = t.find("*/", p)) != std::string::npos;) t.replace(p, 2, "* /");
      return pad(ind) + "/* " + t + " */\n";
    }
    case Stmt::Seq: {
      std::string out;
      for (auto& x : s.items) out += stmt(*x, ind);
      return out;
    }
    case Stmt::For: {
      // a loop of no iterations: the counter is unsigned, so `i <= -1` would never be false
      if (s.to < s.from) return pad(ind) + "/* empty loop " + s.index + " */\n";
      if (s.from < 0) throw Error(-4, "b200ir: loop '" + s.index + "' starts below zero");
      const char* it = large_models ? "unsigned long long" : "unsigned int";
      std::string lo = std::to_string(s.from), hi = std::to_string(s.to);
      std::string head;
      if (!coop_sym.empty() && coop_sym == s.index) {
        // cooperative reduction: the lanes of a warp stride over this loop
        head = pad(ind) + "for (" + it + " " + s.index + " = " + lo + " + b200_lane; " + s.index + " <= " + hi + "; " +
               s.index + " += 32) {\n";
      } else {
        head = (unroll_loops ? "#pragma unroll\n" : std::string()) + pad(ind) + "for (" + it + " " + s.index + " = " + lo + "; " +
               s.index + " <= " + hi + "; ++" + s.index + ") {\n";
      }
      return head + stmt(*s.body, ind + 2) + pad(ind) + "}\n";
    }
    case Stmt::ZeroOut: {
      const Tnode& t = P.tn(s.tn);
      used_nodes.insert(s.tn);
      std::string n = std::to_string(t.num_elems());
      std::string v = "b200_z" + std::to_string(tmp_counter++);
      return pad(ind) + "for (unsigned int " + v + " = 0; " + v + " < " + n + "; ++" + v + ") " + t.ident + "[" + v +
             "] = " + storage_zero(t.prec) + ";\n";
    }
    case Stmt::Set: {
      const Tnode& t = P.tn(s.tn);
      if (t.mode == Mode::Virtual) throw Error(-3, "b200ir: write to virtual node '" + t.ident + "'");
      if (s.vec_len > 0) {
        // C_syntax (arrayjit/lib/c_syntax.ml:548-592): one evaluation of the argument, then one
        // store per element; a Fixed last index advances, any other gets "+ i" on the offset
        if (pair) throw Error(-4, "pair emission of a vector store");
        const char* fn = nullptr;
        int want = 0;
        switch (t.prec) {
          case Prec::Single: fn = "b200_uniform_single("; want = 4; break;
          case Prec::Double: fn = "b200_uniform_double("; want = 2; break;
          case Prec::Int32: fn = "b200_uniform_int32("; want = 4; break;
          case Prec::Int64: fn = "b200_uniform_int64("; want = 2; break;
          case Prec::Bfloat16: fn = "b200_uniform_bfloat16("; want = 8; break;
          case Prec::Half: fn = "b200_uniform_half("; want = 8; break;
          case Prec::Fp8:
          case Prec::Byte: fn = "b200_uniform_byte("; want = 16; break;
          default: throw Error(-4, "uint4x32_to_prec_uniform into an unsupported precision");
        }
        if (s.vec_len != want && s.vec_len != 1) throw Error(-3, "b200ir: vector length does not match the precision");
        if (s.arg_prec != Prec::Uint4x32) throw Error(-4, "uint4x32_to_prec_uniform of a non-uint4x32 argument");
        Res v = scalar(s.arg_prec, *s.value);
        used_nodes.insert(s.tn);
        const std::string tmp = "b200_vec" + std::to_string(tmp_counter++);
        std::string out = pad(ind) + "{\n" + emit_defs(v.defs, ind + 2) + pad(ind + 2) + "const b200_u4x32 " + tmp + " = " + v.expr + ";\n";
        for (int i = 0; i < s.vec_len; ++i) {
          std::string off;
          if (!s.idcs.empty() && s.idcs.back().kind == Index::Fixed) {
            Indices el = s.idcs;
            el.back().fixed += i;
            off = offset(el, t.dims);
          } else {
            off = offset(s.idcs, t.dims) + " + " + std::to_string(i);
          }
          out += pad(ind + 2) + t.ident + "[" + off + "] = " + fn + tmp + ", " + std::to_string(i) + ");\n";
        }
        return out + pad(ind) + "}\n";
      }
      if (pair) {
        auto prd = set_redirect.find(s.tn);
        const bool redirected = prd != set_redirect.end() && same_indices(prd->second.first, s.idcs);
        if (!redirected) {
          // a store to memory: only of a pair that lies side by side (checked by the caller)
          bool contiguous = pair_vector_loads && !s.idcs.empty() && s.idcs.back().kind == Index::Iter &&
                            s.idcs.back().sym == pair_sym && t.dims.back() % 2 == 0;
          for (size_t a = 0; contiguous && a + 1 < s.idcs.size(); ++a)
            if (s.idcs[a].uses(pair_sym)) contiguous = false;
          if (!contiguous) throw Error(-4, "pair emission of a store to memory");
        }
        std::string code;
        const std::string v = pair_scalar(t.prec, *s.value, code);
        used_nodes.insert(s.tn);
        if (redirected) return code + pad(ind) + prd->second.second + " = " + v + ";\n";
        return code + pad(ind) + "*(" + pair_type(t.prec) + "*)(" + t.ident + " + " + offset(s.idcs, t.dims) + ") = " + v + ";\n";
      }
      Res v = scalar(t.prec, *s.value);
      used_nodes.insert(s.tn);
      std::string a = t.ident + "[" + offset(s.idcs, t.dims) + "] = " + store_wrap(t.prec, v.expr) + ";\n";
      auto rd = set_redirect.find(s.tn);
      if (rd != set_redirect.end() && same_indices(rd->second.first, s.idcs)) a = rd->second.second + " = " + v.expr + ";\n";
      if (v.defs.empty()) return pad(ind) + a;
      return pad(ind) + "{\n" + emit_defs(v.defs, ind + 2) + pad(ind + 2) + a + pad(ind) + "}\n";
    }
    case Stmt::SetLocal: {
      Prec p = P.tn(s.tn).prec;
      Res v = scalar(p, *s.value);
      auto sub = scope_subst.find(s.scope_id);
      std::string a = (sub != scope_subst.end() ? sub->second : scope_name(s.scope_id, s.tn)) + " = " + v.expr + ";\n";
      if (v.defs.empty()) return pad(ind) + a;
      return pad(ind) + "{\n" + emit_defs(v.defs, ind + 2) + pad(ind + 2) + a + pad(ind) + "}\n";
    }
    case Stmt::DeclareLocal: {
      Prec p = P.tn(s.tn).prec;
      return pad(ind) + rtype(p) + " " + scope_name(s.scope_id, s.tn) + (s.needs_init ? " = " + constant(0.0, p) : "") + ";\n";
    }
  }
  return "";
}

// ------------------------------------------------------------------------- pair mode

namespace {
std::string pair_lo(Prec p, const std::string& v) {
  if (p == Prec::Single) return v + ".x";
  return (p == Prec::Bfloat16 ? "b200_bf2_lo(" : "b200_hf2_lo(") + v + ")";
}
std::string pair_hi_of(Prec p, const std::string& v) {
  if (p == Prec::Single) return v + ".y";
  return (p == Prec::Bfloat16 ? "b200_bf2_hi(" : "b200_hf2_hi(") + v + ")";
}
// a pair of precision p from two float expressions (rounds when p is a 16-bit format)
std::string pair_make(Prec p, const std::string& lo, const std::string& hi) {
  if (p == Prec::Single) return "b200_f2{" + lo + ", " + hi + "}";
  return (p == Prec::Bfloat16 ? "b200_bf2_pack(" : "b200_hf2_pack(") + lo + ", " + hi + ")";
}
const char* pair_suffix(Prec p) { return p == Prec::Bfloat16 ? "bf2" : "hf2"; }
}  // namespace

bool Emitter::pair_supported(const Scalar& e) const {
  switch (e.kind) {
    case Scalar::Const: return true;
    case Scalar::Get: if (!pair_prec(P.tn(e.tn).prec)) return false; break;
    case Scalar::LocalScope:
    case Scalar::GetLocal:
      return scope_subst.count(e.scope_id) != 0 && pair_prec(P.tn(e.tn).prec);
    case Scalar::Bin:
    case Scalar::Un:
    case Scalar::Tern: break;
    default: return false;
  }
  for (auto& a : e.args) {
    if (!pair_prec(a.prec)) return false;
    if (!pair_supported(*a.s)) return false;
  }
  return true;
}

std::string Emitter::pair_tmp(Prec p, const std::string& init, std::string& code) {
  const std::string n = "b200_t" + std::to_string(tmp_counter++);
  code += std::string("      const ") + pair_type(p) + " " + n + " = " + init + ";\n";
  return n;
}

std::string Emitter::pair_convert(Prec from, Prec to, const std::string& v, std::string& code) {
  if (from == to) return v;
  return pair_tmp(to, pair_make(to, pair_lo(from, v), pair_hi_of(from, v)), code);
}

std::string Emitter::pair_scalar(Prec prec, const Scalar& e, std::string& code) {
  if (!pair_prec(prec)) throw Error(-4, "pair emission of an unsupported precision");
  switch (e.kind) {
    case Scalar::LocalScope:
    case Scalar::GetLocal: {
      auto sub = scope_subst.find(e.scope_id);
      if (sub == scope_subst.end()) throw Error(-4, "pair emission of a local scope");
      return pair_convert(P.tn(e.tn).prec, prec, sub->second, code);
    }
    case Scalar::Const: {
      if (prec == Prec::Single) {
        const std::string c = constant(e.cval, prec);
        return "b200_f2{" + c + ", " + c + "}";
      }
      char buf[32];
      const unsigned int b = lowp_bits(e.cval, prec);
      snprintf(buf, sizeof buf, "0x%08xu", b | (b << 16));
      return buf;
    }
    case Scalar::Get: {
      const Tnode& t = P.tn(e.tn);
      auto f = forwarded.find(e.tn);
      if (f != forwarded.end() && same_indices(f->second.first, e.idcs)) return pair_convert(t.prec, prec, f->second.second, code);
      if (t.mode == Mode::Virtual) throw Error(-3, "b200ir: read of virtual node '" + t.ident + "'");
      used_nodes.insert(e.tn);
      for (auto& lt : load_tiles)
        if (lt.tn == e.tn && same_indices(lt.idcs, e.idcs)) return pair_convert(t.prec, prec, lt.expr, code);
      ++direct_reads;
      const std::string off0 = offset(e.idcs, t.dims);
      {
        // the pair lies side by side in memory when the pair symbol is the last index and nothing else;
        // it is then one 4- or 8-byte load (pair symbols are even and rows of even length keep it aligned)
        bool contiguous = pair_vector_loads && !e.idcs.empty() && e.idcs.back().kind == Index::Iter &&
                          e.idcs.back().sym == pair_sym && t.dims.back() % 2 == 0;
        for (size_t a = 0; contiguous && a + 1 < e.idcs.size(); ++a)
          if (e.idcs[a].uses(pair_sym)) contiguous = false;
        if (contiguous) {
          const std::string v = pair_tmp(t.prec, std::string("*(const ") + pair_type(t.prec) + "*)(" + t.ident + " + " + off0 + ")", code);
          return pair_convert(t.prec, prec, v, code);
        }
      }
      pair_hi = true;
      const std::string off1 = offset(e.idcs, t.dims);
      pair_hi = false;
      const std::string a = t.ident + "[" + off0 + "]", b = t.ident + "[" + off1 + "]";
      std::string v;
      if (t.prec == Prec::Single) v = pair_tmp(t.prec, "b200_f2{" + a + ", " + (off0 == off1 ? a : b) + "}", code);
      else if (off0 == off1) v = pair_tmp(t.prec, "b200_dup16(" + a + ")", code);
      else v = pair_tmp(t.prec, "((unsigned int)" + a + " | ((unsigned int)" + b + " << 16))", code);
      return pair_convert(t.prec, prec, v, code);
    }
    case Scalar::Bin: {
      if (e.op == "arg1") return pair_scalar(prec, *e.args[0].s, code);
      if (e.op == "arg2") return pair_scalar(prec, *e.args[1].s, code);
      if (e.op == "pow" && e.args[1].s->kind == Scalar::Const && (e.args[1].s->cval == 2.0 || e.args[1].s->cval == 3.0)) {
        const std::string a = pair_scalar(prec, *e.args[0].s, code);
        const bool cube = e.args[1].s->cval == 3.0;
        if (lowp(prec)) {
          // one rounding of the float power, as the scalar form does
          const std::string fn = cube ? "b200_pow3(" : "b200_pow2(";
          return pair_tmp(prec, pair_make(prec, fn + pair_lo(prec, a) + ")", fn + pair_hi_of(prec, a) + ")"), code);
        }
        const std::string fn = cube ? "b200_pow3(" : "b200_pow2(";
        return pair_tmp(prec, "b200_f2{" + fn + a + ".x), " + fn + a + ".y)}", code);
      }
      const std::string a = pair_scalar(prec, *e.args[0].s, code), b = pair_scalar(prec, *e.args[1].s, code);
      if (lowp(prec) && (e.op == "add" || e.op == "sub" || e.op == "mul" || e.op == "max" || e.op == "min"))
        return pair_tmp(prec, std::string("b200_") + pair_suffix(prec) + "_" + e.op + "(" + a + ", " + b + ")", code);
      return pair_tmp(prec,
                      pair_make(prec, binop_plain(Prec::Single, e.op, pair_lo(prec, a), pair_lo(prec, b)),
                                binop_plain(Prec::Single, e.op, pair_hi_of(prec, a), pair_hi_of(prec, b))),
                      code);
    }
    case Scalar::Un: {
      const std::string a = pair_scalar(prec, *e.args[0].s, code);
      if (e.op == "id") return a;
      if (lowp(prec)) {
        if (e.op == "neg") return pair_tmp(prec, "(" + a + " ^ 0x80008000u)", code);
        if (e.op == "relu") return pair_tmp(prec, std::string("b200_") + pair_suffix(prec) + "_max(" + a + ", 0u)", code);
        auto one = [&](const std::string& x) {
          if (e.op == "tanh") return "b200_tanh_fast(" + x + ")";
          if (e.op == "exp") return "__expf(" + x + ")";
          if (e.op == "log") return "__logf(" + x + ")";
          return unop_plain(Prec::Single, e.op, x);
        };
        return pair_tmp(prec, pair_make(prec, one(pair_lo(prec, a)), one(pair_hi_of(prec, a))), code);
      }
      return pair_tmp(prec, "b200_f2{" + unop_plain(prec, e.op, a + ".x") + ", " + unop_plain(prec, e.op, a + ".y") + "}", code);
    }
    case Scalar::Tern: {
      if (e.op == "where") {
        const Prec cp = e.args[0].prec;
        const std::string c = pair_scalar(cp, *e.args[0].s, code);
        const std::string a = pair_scalar(prec, *e.args[1].s, code), b = pair_scalar(prec, *e.args[2].s, code);
        const std::string c0 = "(" + pair_lo(cp, c) + " != 0)", c1 = "(" + pair_hi_of(cp, c) + " != 0)";
        if (prec == Prec::Single)
          return pair_tmp(prec, "b200_f2{" + c0 + " ? " + a + ".x : " + b + ".x, " + c1 + " ? " + a + ".y : " + b + ".y}", code);
        return pair_tmp(prec, "b200_sel16x2(" + c0 + ", " + c1 + ", " + a + ", " + b + ")", code);
      }
      const std::string a = pair_scalar(prec, *e.args[0].s, code), b = pair_scalar(prec, *e.args[1].s, code),
                        c = pair_scalar(prec, *e.args[2].s, code);
      return pair_tmp(prec,
                      pair_make(prec, ternop_plain(Prec::Single, e.op, pair_lo(prec, a), pair_lo(prec, b), pair_lo(prec, c)),
                                ternop_plain(Prec::Single, e.op, pair_hi_of(prec, a), pair_hi_of(prec, b), pair_hi_of(prec, c))),
                      code);
    }
    default: break;
  }
  throw Error(-4, "pair emission of an unsupported scalar");
}

}  // namespace b200
