// CUDA C emission of Low_level statements and scalars.
//
// The arithmetic contract is the cc backend's (arrayjit/lib/c_syntax.ml:441-855 with the
// operator tables of arrayjit/lib/ops.ml:579-863 and the compute-in-float rule for
// bf16/half of arrayjit/lib/cc_backend.ml:169-322): every homogeneous operation converts
// its arguments to the RESULT precision first, `where` keeps the precision of its
// condition, constants are doubles converted to the context precision, offsets are
// row-major.  Differences from the C text, none of which changes a result beyond the last
// bit: float contexts use float literals (the C text writes `0.0`/`1.0` and lets the
// compiler fold them), and indices are `unsigned`.
#pragma once
#include <map>
#include <set>
#include <string>
#include <utility>
#include <vector>

#include "ir.hpp"

namespace b200 {

struct Emitter {
  const Program& P;
  bool large_models = false;
  // scope ids whose Local_scope is replaced by a ready expression (the accumulator a
  // contraction kernel hands to its epilogue)
  std::map<int, std::string> scope_subst;
  // (node id) -> expression holding the value just stored at the position of the current
  // parallel iteration; lets a fused consumer read a producer's value from a register
  std::map<int, std::pair<Indices, std::string>> forwarded;
  // (node id) -> lvalue that receives a Set at exactly these indices instead of memory (the
  // register tile of a contraction epilogue; the caller stores the tile afterwards)
  std::map<int, std::pair<Indices, std::string>> set_redirect;
  // reads that were pre-loaded into a register tile: a Get of `tn` at exactly `idcs` becomes `expr`
  struct LoadTile {
    int tn;
    Indices idcs;
    std::string expr;
  };
  std::vector<LoadTile> load_tiles;
  // Row forwarding (the row followers of a contraction epilogue): a thread holds one whole output
  // row of `tn` in registers -- `name[0 .. N)` when `n_axis` >= 0, the scalar `name` otherwise.  A
  // Get of `tn` whose other indices equal `idcs` (after renaming its symbols through `row_ren`)
  // and whose index on `n_axis` is a loop symbol or a fixed position reads `name[that index]`.
  struct RowForward {
    int tn;
    Indices idcs;
    int n_axis;
    std::string name;
    std::string index_shift;   // appended to the index on n_axis ("" or e.g. " - b200_t0": the array holds a slice)
    std::string fixed_index;   // non-empty: the register index of the element the current loop is at, whatever the symbol
  };
  std::vector<RowForward> row_forwards;
  std::map<std::string, std::string> row_ren;
  bool unroll_loops = false;   // `#pragma unroll` before every emitted loop (register arrays stay registers)
  // divisors prepared once for many numerators: emitted text of the divisor -> name of a b200_divisor
  // variable in scope; a single-precision (or 16-bit) division by exactly that text uses it
  std::map<std::string, std::string> divisor_vars;
  // when set, the emitted text of every single-precision divisor is appended here (a caller that
  // wants to prepare row-invariant divisors emits once to see them)
  std::vector<std::string>* divisor_probe = nullptr;
  // nodes read through another name (a copy staged in shared memory)
  std::map<int, std::string> node_alias;
  // nodes whose loads may use the read-only data path
  std::set<int> readonly_nodes;
  // cooperative reductions: scope id -> lane-strided loop symbol (see compile.cpp)
  std::string coop_sym;
  std::set<int> used_nodes;
  bool uses_statics = false, uses_merge = false;
  int tmp_counter = 0;
  int direct_reads = 0;   // reads emitted as plain memory accesses (not served by a register tile)

  explicit Emitter(const Program& p) : P(p) {}

  static const char* ctype(Prec p);   // storage type of a node
  static const char* rtype(Prec p);   // type of a value of that precision inside an expression
  static std::string load_wrap(Prec p, const std::string& storage_expr);
  static std::string store_wrap(Prec p, const std::string& value_expr);
  std::string storage_zero(Prec p);
  static std::pair<std::string, std::string> convert(Prec from, Prec to);
  std::string index(const Index& ix);
  std::string offset(const Indices& idcs, const std::vector<int64_t>& dims, int dyn_axis = -1,
                     const std::string& dyn_doc = "");
  std::string scope_name(int scope_id, int tn) const;
  std::string node_name(int tn) const;

  struct Res {
    std::vector<std::pair<int, std::string>> defs;
    std::string expr;
  };
  Res scalar(Prec prec, const Scalar& s);
  std::string stmt(const Stmt& s, int indent);
  std::string constant(double c, Prec prec);
  static bool reads_scope_before_set(int scope_id, int tn, const Stmt& body);

  // ---- pair mode: every value is TWO neighbouring elements along `pair_sym` (sym and sym + 1).
  // Single values are a `b200_f2`, bf16 / half values one 32-bit word holding both (element
  // `sym` in the low half), so that add / sub / mul / min / max / neg / fma run as one packed
  // instruction and a float pair is rounded by one packed conversion.  For two operands that are
  // values of the 16-bit format, the packed add / sub / mul round the exact result once; the
  // float operation followed by a rounding gives the same bits, because whenever the exact
  // result does not fit a float the smaller operand is far below half a unit in the last place
  // of the larger one and both roundings return the larger operand.
  bool pair = false;
  std::string pair_sym;
  bool pair_hi = false;   // while true, index() spells pair_sym as (pair_sym + 1u)
  bool pair_vector_loads = false;  // the pair symbol takes even values only: side-by-side pairs are one access
  static bool pair_prec(Prec p) { return p == Prec::Single || p == Prec::Bfloat16 || p == Prec::Half; }
  static const char* pair_type(Prec p) { return p == Prec::Single ? "b200_f2" : "unsigned int"; }
  // whether `s` can be emitted in pair mode (given the scopes that are substituted)
  bool pair_supported(const Scalar& s) const;
  // emits definitions of temporaries into `code` and returns the name / expression of the value
  std::string pair_scalar(Prec prec, const Scalar& s, std::string& code);
  std::string pair_convert(Prec from, Prec to, const std::string& v, std::string& code);
  std::string pair_tmp(Prec p, const std::string& init, std::string& code);

  std::string binop(Prec prec, const std::string& op, const std::string& a, const std::string& b);
  std::string unop(Prec prec, const std::string& op, const std::string& a);
  std::string ternop(Prec prec, const std::string& op, const std::string& a, const std::string& b,
                     const std::string& c);
};

}  // namespace b200
