// b200ir: the serialised form of arrayjit's `Low_level.optimized` that crosses the C ABI.
//
// The node kinds are the constructors of `Low_level.t` / `scalar_t`
// (arrayjit/lib/low_level.mli:22-68) and `Indexing.axis_index`
// (arrayjit/lib/indexing.ml:104-120); the per-node facts are those of `traced_array`
// (low_level.mli:104-130) plus the memory class `C_syntax.compile_proc` derives
// (arrayjit/lib/c_syntax.ml:1028-1043).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace b200 {

struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

enum class Prec { Byte, Uint16, Int32, Uint32, Int64, Uint64, Uint4x32, Half, Bfloat16, Fp8, Single, Double };
Prec prec_of_string(const std::string& s);
const char* prec_name(Prec p);
int prec_bytes(Prec p);
inline bool is_int_prec(Prec p) {
  return p == Prec::Byte || p == Prec::Uint16 || p == Prec::Int32 || p == Prec::Uint32 ||
         p == Prec::Int64 || p == Prec::Uint64 || p == Prec::Fp8;
}

enum class Mode { Virtual, Local, Ctx, Global };

struct Tnode {
  int id = 0;
  std::string ident;
  Prec prec = Prec::Single;
  std::vector<int64_t> dims;
  Mode mode = Mode::Ctx;
  bool zero_init = false;
  bool read_only = false;
  int64_t num_elems() const {
    int64_t n = 1;
    for (auto d : dims) n *= d;
    return n;
  }
  int64_t bytes() const { return num_elems() * prec_bytes(prec); }
  bool is_param() const { return mode == Mode::Ctx || mode == Mode::Global; }
};

// ---- indices
struct Index {
  enum Kind { Fixed, Iter, Affine, SubAxis } kind = Fixed;
  int64_t fixed = 0;                                   // Fixed value / Affine offset
  std::string sym;                                     // Iter
  std::vector<std::pair<int64_t, std::string>> terms;  // Affine
  bool uses(const std::string& s) const {
    if (kind == Iter) return sym == s;
    if (kind == Affine)
      for (auto& t : terms)
        if (t.second == s) return true;
    return false;
  }
};
using Indices = std::vector<Index>;

// ---- scalars and statements
struct Stmt;
using StmtP = std::shared_ptr<Stmt>;
struct Scalar;
using ScalarP = std::shared_ptr<Scalar>;

struct Arg {
  ScalarP s;
  Prec prec;
};

struct Scalar {
  enum Kind { LocalScope, GetLocal, Get, GetDyn, GetMerge, Tern, Bin, Un, Const, ConstBits, EmbedIdx } kind;
  // LocalScope / GetLocal
  int scope_id = 0;
  int tn = 0;  // tensor node id (scope's node, or the node read)
  StmtP body;
  Indices idcs;  // Get / GetDyn / GetMerge indices ; LocalScope orig_indices
  int dyn_axis = -1;
  std::string op;
  std::vector<Arg> args;
  double cval = 0;
  int64_t bits = 0;
  Index idx;
};

struct Stmt {
  enum Kind { Noop, Comment, Seq, For, ZeroOut, Set, SetLocal, DeclareLocal } kind;
  std::string text;  // Comment
  std::vector<StmtP> items;
  std::string index;  // For
  int64_t from = 0, to = 0;
  StmtP body;
  int tn = 0;
  Indices idcs;
  ScalarP value;
  int scope_id = 0;
  bool needs_init = false;
  // Set_from_vec is a Set whose value is a vector operation: `vec_len` results go to `vec_len`
  // consecutive elements starting at idcs; `value` is the operation's argument at `arg_prec`
  int vec_len = 0;
  std::string vec_op;
  Prec arg_prec = Prec::Single;
};

struct StaticSym {
  std::string sym;
  int64_t range = -1;  // -1: none
};

struct Program {
  std::string name;
  std::vector<Tnode> tnodes;  // declaration order
  std::map<int, size_t> tn_index;
  std::vector<StaticSym> statics;
  int merge_node = -1;
  StmtP body;
  const Tnode& tn(int id) const {
    auto it = tn_index.find(id);
    if (it == tn_index.end()) throw Error(-3, "b200ir: unknown tensor node id " + std::to_string(id));
    return tnodes[it->second];
  }
};

// Parses b200ir text (version 1).  Throws Error(-3, ...) on malformed input.
Program parse_program(const char* text, size_t len);

}  // namespace b200
