// Routine compilation: cut the body into stages, find the parallel loops of each stage and
// generate its kernel.  See compile.hpp.
//
// The reference runs a routine as ONE sequential function (cc: arrayjit/lib/cc_backend.ml:325-343;
// cuda: one thread of one block, arrayjit/lib/cuda_backend.ml:357-360,1043).  Here every
// top-level loop nest (`loop_accum` emits one per assignment, arrayjit/lib/assignments.ml:311-488)
// becomes a kernel whose threads own disjoint iterations of the nest's independent loops.
#include "compile.hpp"

#include <algorithm>
#include <cmath>
#include <functional>
#include <set>
#include <sstream>

#include "emit.hpp"

namespace b200 {

bool match_attention(const Program& P, const std::vector<StmtP>& flat, size_t at, const CompileOptions& opt, int* n_absorbed,
                     Stage* out);
std::string attn_translation_unit(const Program& P, Stage& st, const std::string& kernel_name);
bool match_gemm(const Program& P, const std::vector<LoopDim>& nest, const Stmt& body, bool zeroed_before,
                const CompileOptions& opt, const std::vector<Follower>& followers, int* n_fused,
                Stage* out);  // gemm_match.cpp
std::string gemm_translation_unit(const Program& P, Stage& st, const std::string& kernel_name,
                                  const CompileOptions& opt);

namespace {

// ---- walking helpers
void walk_scalar(const Scalar& e, const std::function<void(const Scalar&)>& fs,
                 const std::function<void(const Stmt&)>& ft);
void walk_stmt(const Stmt& s, const std::function<void(const Scalar&)>& fs, const std::function<void(const Stmt&)>& ft) {
  ft(s);
  switch (s.kind) {
    case Stmt::Seq:
      for (auto& x : s.items) walk_stmt(*x, fs, ft);
      break;
    case Stmt::For: walk_stmt(*s.body, fs, ft); break;
    case Stmt::Set:
    case Stmt::SetLocal: walk_scalar(*s.value, fs, ft); break;
    default: break;
  }
}
void walk_scalar(const Scalar& e, const std::function<void(const Scalar&)>& fs,
                 const std::function<void(const Stmt&)>& ft) {
  fs(e);
  if (e.kind == Scalar::LocalScope) walk_stmt(*e.body, fs, ft);
  for (auto& a : e.args) walk_scalar(*a.s, fs, ft);
}

// Is loop symbol `s` safe to run in parallel over `body`?  Sufficient condition: every
// node written in the body is written only at positions that carry `s` as a plain iterator
// on one fixed axis, and every read of such a node carries `s` on that same axis — so
// distinct values of `s` touch disjoint slices of everything that is written.
bool parallel_safe(const std::string& s, const Stmt& body) {
  std::map<int, int> axis_of;  // written node -> axis that carries s
  std::map<int, Index> index_of;  // written node -> the index on that axis
  bool ok = true;
  // an index is one-to-one in s when it is s itself or c * s + fixed with c != 0 (a padded
  // node addressed past its margin)
  auto one_to_one = [&](const Index& ix) {
    return (ix.kind == Index::Iter && ix.sym == s) ||
           (ix.kind == Index::Affine && ix.terms.size() == 1 && ix.terms[0].second == s && ix.terms[0].first != 0);
  };
  auto same_index = [](const Index& a, const Index& b) {
    return a.kind == b.kind && a.sym == b.sym && a.fixed == b.fixed && a.terms == b.terms;
  };
  auto axis_with = [&](const Indices& idcs) {
    for (size_t a = 0; a < idcs.size(); ++a)
      if (one_to_one(idcs[a])) return (int)a;
    return -1;
  };
  walk_stmt(
      body, [](const Scalar&) {},
      [&](const Stmt& st) {
        if (st.kind == Stmt::ZeroOut) ok = false;
        if (st.kind == Stmt::Set) {
          int a = axis_with(st.idcs);
          if (st.vec_len > 0 && a >= 0 && st.idcs[a].kind == Index::Affine) a = -1;  // judged by the rule below
          if (a < 0 && st.vec_len > 0 && !st.idcs.empty()) {
            // a vector store whose last index is c * s (+ fixed) with c >= the vector length
            // writes disjoint runs for distinct s
            const Index& last = st.idcs.back();
            if (last.kind == Index::Affine && last.terms.size() == 1 && last.terms[0].second == s &&
                last.terms[0].first >= st.vec_len)
              a = (int)st.idcs.size() - 1;
          } else if (a >= 0 && st.vec_len > 1 && a == (int)st.idcs.size() - 1) {
            a = -1;  // runs of neighbouring elements would overlap
          }
          if (a < 0) { ok = false; return; }
          // the symbol must not appear on any other axis of the write
          for (size_t k = 0; k < st.idcs.size(); ++k)
            if ((int)k != a && st.idcs[k].uses(s)) ok = false;
          auto it = axis_of.find(st.tn);
          if (it == axis_of.end()) { axis_of[st.tn] = a; index_of[st.tn] = st.idcs[a]; }
          else if (it->second != a || !same_index(index_of[st.tn], st.idcs[a])) ok = false;
        }
      });
  if (!ok) return false;
  walk_stmt(
      body,
      [&](const Scalar& e) {
        if (e.kind == Scalar::Get || e.kind == Scalar::GetDyn) {
          auto it = axis_of.find(e.tn);
          if (it == axis_of.end()) return;
          if (e.kind == Scalar::GetDyn) { ok = false; return; }
          int a = it->second;
          if (a >= (int)e.idcs.size() || !same_index(e.idcs[a], index_of[e.tn])) ok = false;
          for (size_t k = 0; k < e.idcs.size(); ++k)
            if ((int)k != a && e.idcs[k].uses(s)) ok = false;
        }
      },
      [](const Stmt&) {});
  return ok;
}

// `t[p] := fma(a, b, t[p])` or `t[p] := t[p] + term` (either order) where neither a, b nor the
// term read t or hold a local scope.
bool accumulates_into_self(const Stmt& set) {
  if (set.kind != Stmt::Set || !set.value) return false;
  const Scalar& v = *set.value;
  auto is_self = [&](const Scalar& e) {
    if (e.kind != Scalar::Get || e.tn != set.tn || e.idcs.size() != set.idcs.size()) return false;
    for (size_t i = 0; i < e.idcs.size(); ++i)
      if (e.idcs[i].kind != set.idcs[i].kind || e.idcs[i].sym != set.idcs[i].sym || e.idcs[i].fixed != set.idcs[i].fixed ||
          e.idcs[i].terms != set.idcs[i].terms)
        return false;
    return true;
  };
  auto plain = [&](const Scalar& e) {
    bool ok = true;
    walk_scalar(e, [&](const Scalar& x) {
      if ((x.kind == Scalar::Get || x.kind == Scalar::GetDyn) && x.tn == set.tn) ok = false;
      if (x.kind == Scalar::LocalScope) ok = false;
    }, [](const Stmt&) {});
    return ok;
  };
  if (v.kind == Scalar::Tern && v.op == "fma")
    return is_self(*v.args[2].s) && plain(*v.args[0].s) && plain(*v.args[1].s);
  if (v.kind == Scalar::Bin && v.op == "add")
    return (is_self(*v.args[0].s) && plain(*v.args[1].s)) || (is_self(*v.args[1].s) && plain(*v.args[0].s));
  return false;
}

bool body_has_set(const Stmt& s) {
  bool any = false;
  walk_stmt(s, [](const Scalar&) {}, [&](const Stmt& st) {
    if (st.kind == Stmt::Set || st.kind == Stmt::ZeroOut) any = true;
  });
  return any;
}

// Does the statement tree mention a function-scope scalar local (declared outside it)?
void collect_scopes(const Stmt& s, std::set<std::pair<int, int>>& declared, std::set<std::pair<int, int>>& used) {
  walk_stmt(
      s,
      [&](const Scalar& e) {
        if (e.kind == Scalar::LocalScope) declared.insert({e.scope_id, e.tn});
        if (e.kind == Scalar::GetLocal) used.insert({e.scope_id, e.tn});
      },
      [&](const Stmt& st) {
        if (st.kind == Stmt::DeclareLocal) declared.insert({st.scope_id, st.tn});
        if (st.kind == Stmt::SetLocal) used.insert({st.scope_id, st.tn});
      });
}

// Cooperative row reduction: the stage's body is `Set t[..] := E` where E holds Local_scope
// reductions `v := neutral; for k { v := v (+|max|min) f(k) }` over loops long enough that a
// warp per output element pays.  Returns the lane-strided symbol or "".
struct CoopInfo {
  std::string sym;
  int width = 32;  // threads cooperating on one output element
  int grid_blocks = 0;  // >0: two-kernel grid-wide reduction with this many blocks in pass 1
  std::vector<std::pair<int, std::string>> scopes;  // (scope id, combine op)
};

bool accum_form(const Stmt& st, int sid, int tn, std::string* op) {
  // Set_local(id, Binop(op, Get_local id, x)) | Binop(op, x, Get_local id) | FMA(a, b, Get_local id)
  if (st.kind != Stmt::SetLocal || st.scope_id != sid || st.tn != tn) return false;
  const Scalar& v = *st.value;
  auto is_self = [&](const Scalar& e) { return e.kind == Scalar::GetLocal && e.scope_id == sid && e.tn == tn; };
  auto mentions_self = [&](const Scalar& e) {
    bool m = false;
    walk_scalar(e, [&](const Scalar& x) { if (is_self(x)) m = true; }, [](const Stmt&) {});
    return m;
  };
  if (v.kind == Scalar::Tern && v.op == "fma") {
    if (is_self(*v.args[2].s) && !mentions_self(*v.args[0].s) && !mentions_self(*v.args[1].s)) {
      *op = "add";
      return true;
    }
    return false;
  }
  if (v.kind == Scalar::Bin && (v.op == "add" || v.op == "max" || v.op == "min")) {
    if (is_self(*v.args[0].s) && !mentions_self(*v.args[1].s)) { *op = v.op; return true; }
    if (is_self(*v.args[1].s) && !mentions_self(*v.args[0].s)) { *op = v.op; return true; }
  }
  return false;
}

}  // namespace

double GemmPlan::flops() const {
  double f = 2.0 * (double)m.extent * (double)n.extent * (double)k.extent;
  for (auto& b : batch) f *= (double)b.extent;
  return f;
}

std::string Code::describe() const {
  std::ostringstream o;
  o << "{\"name\":\"" << prog.name << "\",\"stages\":[";
  for (size_t i = 0; i < stages.size(); ++i) {
    const Stage& s = stages[i];
    if (i) o << ",";
    o << "{\"kind\":\"" << (s.kind == Stage::Memset ? "memset" : s.kind == Stage::Gemm ? "gemm" : s.kind == Stage::Attn ? "attention" : "generic") << "\"";
    o << ",\"kernel\":\"" << s.kernel << "\",\"total\":" << s.total << ",\"coop\":" << s.coop;
    if (s.kind == Stage::Gemm) {
      o << ",\"m\":" << s.gemm.m.extent << ",\"n\":" << s.gemm.n.extent << ",\"k\":" << s.gemm.k.extent;
      int64_t b = 1;
      for (auto& d : s.gemm.batch) b *= d.extent;
      o << ",\"batch\":" << b << ",\"a_kmajor\":" << (s.gemm.a_kmajor ? 1 : 0) << ",\"b_kmajor\":" << (s.gemm.b_kmajor ? 1 : 0)
        << ",\"accumulate\":" << (s.gemm.accumulate ? 1 : 0) << ",\"flops\":" << s.gemm.flops();
    }
    if (s.kind == Stage::Attn) {
      const AttnPlan& a = s.attn;
      // both contractions: queries x keys x head dimension, twice
      o << ",\"queries\":" << a.S << ",\"keys\":" << a.T << ",\"head_dim\":" << a.E << ",\"batch\":" << a.B0 * a.B1
        << ",\"flops\":" << 4.0 * (double)(a.B0 * a.B1) * (double)a.S * (double)a.T * (double)a.E;
    }
    if (s.kind != Stage::Memset) {
      // bytes of every node the stage touches, each counted once: the stage's algorithmic traffic
      long long bytes = 0;
      for (auto& a : s.args)
        if (a.kind == KArg::Node) bytes += prog.tn(a.tn).bytes();
      if (s.kind == Stage::Gemm) bytes += prog.tn(s.gemm.a_tn).bytes() + prog.tn(s.gemm.b_tn).bytes();
      if (s.kind == Stage::Attn) bytes += prog.tn(s.attn.q_tn).bytes() + prog.tn(s.attn.k_tn).bytes() + prog.tn(s.attn.v_tn).bytes();
      o << ",\"bytes\":" << bytes;
    } else {
      o << ",\"bytes\":" << prog.tn(s.memset_tn).bytes();
    }
    o << ",\"note\":\"" << s.note << "\"}";
  }
  o << "]}";
  return o.str();
}

namespace {

// What generic_stage knows about a stage before its kernel text is written.
// First statements of every generated kernel: let the next kernel in the stream be placed, then
// wait until the grids before this one have completed and their writes are visible.
static const char* kGridEntry =
    "  asm volatile(\"griddepcontrol.launch_dependents;\");\n  asm volatile(\"griddepcontrol.wait;\" ::: \"memory\");\n";

struct Piece {
  bool fusable = false;
  std::string decomp, body_text;
  std::set<int> used, written;
  bool uses_merge = false;
  // row fusion: the outermost parallel loop ("row") and the work of one of its iterations
  StmtP body;
  std::string row_sym;
  int64_t rows = 0, per_row = 0;
  // warp-per-row fusion: the stage's parallel loops, whether a warp cooperates on each output
  // element (its reductions are warp-wide), whether a thread takes pairs of the innermost loop
  StmtP any_body;
  std::vector<LoopDim> par;
  int coop = 0;
  bool pairs = false;
  int64_t ser_work = 1;
  std::vector<int> staged;   // small read-only nodes the kernel first copies into shared memory
};

struct Builder {
  Code& code;
  const CompileOptions& opt;
  std::ostringstream src;
  int next_kernel = 0;
  int cur_origin = -1;             // index of the top-level statement being planned
  std::map<size_t, Piece> pieces;  // by index into code.stages
  bool pairs_here() const { return opt.enable_pairs && !opt.no_pairs_at.count(cur_origin); }
  bool gemm_at(size_t i) const { return opt.enable_gemm && !opt.no_gemm_at.count((int)i); }

  std::string kernel_name() { return code.prog.name + "_s" + std::to_string(next_kernel++); }

  void emit_params(std::ostringstream& o, Stage& st, const Emitter& em, const std::set<int>& written) {
    // parameters in node declaration order, then the static-index table, then the merge buffer
    bool first = true;
    for (auto& t : code.prog.tnodes) {
      if (!em.used_nodes.count(t.id)) continue;
      if (t.mode == Mode::Virtual) continue;
      if (!first) o << ", ";
      first = false;
      const bool ro = !written.count(t.id);
      o << (ro ? "const " : "") << Emitter::ctype(t.prec) << "* " << (ro ? "__restrict__ " : "") << t.ident;
      st.args.push_back({KArg::Node, t.id});
    }
    if (em.uses_statics) {
      if (!first) o << ", ";
      first = false;
      o << "const unsigned int* __restrict__ b200_statics";
      st.args.push_back({KArg::Statics, -1});
    }
    if (em.uses_merge) {
      if (!first) o << ", ";
      first = false;
      o << "const " << Emitter::ctype(code.prog.tn(code.prog.merge_node).prec) << "* __restrict__ merge_buffer";
      st.args.push_back({KArg::Merge, -1});
    }
  }

  std::string static_prologue(const std::string& body_text, Emitter& em, int ind) {
    // static index symbols are read from the table the launcher fills
    std::string out;
    for (size_t i = 0; i < code.prog.statics.size(); ++i) {
      const std::string& s = code.prog.statics[i].sym;
      // whole-word search
      size_t p = 0;
      bool found = false;
      while ((p = body_text.find(s, p)) != std::string::npos) {
        auto isid = [](char c) { return isalnum((unsigned char)c) || c == '_'; };
        bool l = p == 0 || !isid(body_text[p - 1]);
        bool r = p + s.size() >= body_text.size() || !isid(body_text[p + s.size()]);
        if (l && r) { found = true; break; }
        p += s.size();
      }
      if (found) {
        out += std::string((size_t)ind, ' ') + "const unsigned int " + s + " = b200_statics[" + std::to_string(i) + "];\n";
        em.uses_statics = true;
      }
    }
    return out;
  }

  // Cooperative reduction: the stage's assignment holds Local_scope reductions
  // `v := neutral; for k1 { for k2 .. { v := v (+|max|min) f(k..) } }`.  A group of threads (a
  // warp, or a whole block when there are few outputs and much to reduce) strides over the
  // flattened reduction space of one output element and combines its partial results.
  CoopInfo find_coop(const Stmt& body, int64_t par_total) {
    CoopInfo ci;
    if (!opt.enable_coop) return ci;
    if (body.kind != Stmt::Set) return ci;
    std::vector<const Scalar*> scopes;
    bool nested = false;
    std::function<void(const Scalar&, int)> rec = [&](const Scalar& e, int depth) {
      if (e.kind == Scalar::LocalScope) {
        if (depth > 0) nested = true;
        scopes.push_back(&e);
        walk_stmt(*e.body, [&](const Scalar& x) { if (x.kind == Scalar::LocalScope) nested = true; }, [](const Stmt&) {});
        return;
      }
      for (auto& a : e.args) rec(*a.s, depth);
    };
    rec(*body.value, 0);
    if (scopes.empty() || nested) return ci;
    int64_t extent = -1;
    for (auto* sc : scopes) {
      const Stmt& b = *sc->body;
      const Stmt* loop = nullptr;
      const Stmt* init = nullptr;
      if (b.kind == Stmt::For) loop = &b;
      else if (b.kind == Stmt::Seq && b.items.size() == 2 && b.items[0]->kind == Stmt::SetLocal && b.items[1]->kind == Stmt::For) {
        init = b.items[0].get();
        loop = b.items[1].get();
      } else return CoopInfo{};
      if (init && (init->scope_id != sc->scope_id || init->value->kind != Scalar::Const)) return CoopInfo{};
      int64_t ext = 1;
      const Stmt* inner = loop;
      while (inner->kind == Stmt::For) {
        ext *= inner->to - inner->from + 1;
        inner = inner->body.get();
      }
      std::string op;
      if (!accum_form(*inner, sc->scope_id, sc->tn, &op)) return CoopInfo{};
      Prec p = code.prog.tn(sc->tn).prec;
      if (p != Prec::Single && !(p == Prec::Double && op == "add")) return CoopInfo{};
      // the initial value must be the neutral element of the combine
      double want = op == "add" ? 0.0 : (op == "max" ? -INFINITY : INFINITY);
      if (init && init->value->cval != want) return CoopInfo{};
      if (!init && op != "add") return CoopInfo{};
      if (extent < 0) extent = ext;
      else if (ext != extent) return CoopInfo{};
      ci.scopes.push_back({sc->scope_id, op});
    }
    if (extent < 64) return CoopInfo{};
    ci.sym = "*";
    // few outputs and a long reduction: a whole block per output element
    ci.width = (par_total <= 256 && extent >= 4096) ? 1024 : 32;
    // a single output fed by a very long reduction: many blocks write partial results to
    // scratch and a second, single-block kernel combines them
    if (par_total == 1 && extent >= 32768) {
      ci.width = 1024;
      ci.grid_blocks = (int)std::min<int64_t>(296, (extent + 1023) / 1024);
    }
    return ci;
  }

  // Grid-wide reduction of a single output element in one launch.  Every block reduces a strided
  // slice of each Local_scope's flattened loop space and writes one partial per scope to
  // scratch[scope_index * blocks + block]; the block that takes the last ticket of a counter in
  // scratch (zero at link time, reset here) then combines the partials in block order -- a fixed
  // order, so the result does not depend on scheduling -- and evaluates the assignment.
  void grid_reduce_stage(const StmtP& body, const CoopInfo& ci) {
    const Stmt& set = *body;
    const Tnode& t = code.prog.tn(set.tn);
    const int G = ci.grid_blocks;
    const size_t scratch_off = code.reduce_scratch_bytes;
    const size_t counter_off = (size_t)G * ci.scopes.size() * 8;
    code.reduce_scratch_bytes += counter_off + 8;
    code.reduce_scratch_bytes = (code.reduce_scratch_bytes + 255) & ~(size_t)255;

    Stage a;
    a.kind = Stage::Generic;
    a.kernel = kernel_name();
    a.total = 1;
    a.block = 1024;
    a.coop = 1024;
    a.grid_override = G;

    Emitter ea(code.prog), eb(code.prog);
    ea.large_models = eb.large_models = opt.large_models;
    std::string pass1, pass2;
    int si = 0;
    std::function<void(const Scalar&)> rec = [&](const Scalar& e) {
      if (e.kind == Scalar::LocalScope) {
        std::string op;
        for (auto& s : ci.scopes)
          if (s.first == e.scope_id) op = s.second;
        Prec p = code.prog.tn(e.tn).prec;
        const Stmt& sb = *e.body;
        const Stmt* loop = sb.kind == Stmt::For ? &sb : sb.items[1].get();
        std::vector<LoopDim> red;
        const Stmt* inner = loop;
        while (inner->kind == Stmt::For) {
          red.push_back({inner->index, inner->from, inner->to});
          inner = inner->body.get();
        }
        int64_t total = 1;
        for (auto& d : red) total *= d.extent();
        const std::string name = ea.scope_name(e.scope_id, e.tn);
        const std::string T = Emitter::ctype(p);
        const double neutral = op == "add" ? 0.0 : (op == "max" ? -INFINITY : INFINITY);
        const std::string fn = op == "add" ? "sum" : op;
        const std::string at = "(b200_partials + " + std::to_string((size_t)si * G * 8) + "))";
        const std::string slot = "((" + T + "*)" + at, vslot = "((volatile " + T + "*)" + at;
        pass1 += "  {\n    " + T + " " + name + " = " + ea.constant(neutral, p) + ";\n";
        pass1 += "    for (unsigned long long b200_l = (unsigned long long)blockIdx.x * 1024ull + threadIdx.x; b200_l < " +
                 std::to_string(total) + "ull; b200_l += (unsigned long long)gridDim.x * 1024ull) {\n";
        std::string rem = "b200_l";
        for (size_t i = red.size(); i-- > 0;) {
          const LoopDim& d = red[i];
          std::string ext = std::to_string(d.extent()) + "ull";
          std::string val = i == 0 ? rem : "(" + rem + " % " + ext + ")";
          pass1 += "      const unsigned int " + d.sym + " = (unsigned int)" + val +
                   (d.from ? " + " + std::to_string(d.from) : std::string()) + ";\n";
          if (i != 0) {
            std::string nr = "b200_q" + std::to_string(i);
            pass1 += "      const unsigned long long " + nr + " = " + rem + " / " + ext + ";\n";
            rem = nr;
          }
        }
        pass1 += ea.stmt(*inner, 6);
        pass1 += "    }\n    " + name + " = b200_block_" + fn + "(" + name + ", b200_red);\n";
        pass1 += "    if (threadIdx.x == 0) " + slot + "[blockIdx.x] = " + name + ";\n  }\n";
        // combine: the partials in block order
        pass2 += "  " + T + " " + name + " = " + eb.constant(neutral, p) + ";\n";
        pass2 += "  for (unsigned int b200_i = threadIdx.x; b200_i < " + std::to_string(G) + "u; b200_i += blockDim.x) " + name + " = ";
        if (op == "add") pass2 += name + " + " + vslot + "[b200_i];\n";
        else pass2 += std::string("f") + op + (p == Prec::Double ? "(" : "f(") + name + ", " + vslot + "[b200_i]);\n";
        pass2 += "  " + name + " = b200_block_" + fn + "(" + name + ", b200_red);\n";
        eb.scope_subst[e.scope_id] = name;
        ++si;
        return;
      }
      for (auto& x : e.args) rec(*x.s);
    };
    rec(*set.value);
    Emitter::Res v = eb.scalar(t.prec, *set.value);
    eb.used_nodes.insert(set.tn);
    pass2 += "  if (threadIdx.x == 0) {\n    " + t.ident + "[" + eb.offset(set.idcs, t.dims) + "] = " + Emitter::store_wrap(t.prec, v.expr) +
             ";\n    *b200_ticket = 0u;\n  }\n";

    std::set<int> written = {set.tn};
    Emitter eu(code.prog);
    eu.used_nodes = ea.used_nodes;
    eu.used_nodes.insert(eb.used_nodes.begin(), eb.used_nodes.end());
    eu.uses_merge = ea.uses_merge || eb.uses_merge;
    std::ostringstream ka;
    std::string statics = static_prologue(pass1 + pass2, eu, 2);
    ka << "extern \"C\" __global__ void __launch_bounds__(1024) " << a.kernel << "(";
    emit_params(ka, a, eu, written);
    ka << (a.args.empty() ? "" : ", ") << "unsigned char* b200_partials) {\n" << kGridEntry << "  __shared__ double b200_red[32];\n"
       << "  __shared__ unsigned int b200_last;\n  unsigned int* b200_ticket = (unsigned int*)(b200_partials + " << counter_off << ");\n"
       << statics << pass1
       << "  __threadfence();\n  __syncthreads();\n"
       << "  if (threadIdx.x == 0) b200_last = atomicAdd(b200_ticket, 1u) == gridDim.x - 1u ? 1u : 0u;\n"
       << "  __syncthreads();\n  if (!b200_last) return;\n  __threadfence();\n"
       << pass2 << "}\n\n";
    a.args.push_back({KArg::Scratch, (int)scratch_off});
    src << ka.str();
    a.note = "grid-wide reduction (" + std::to_string(G) + " blocks, the last one combines)";
    a.writes = {set.tn};
    code.stages.push_back(a);
  }

  // Accumulation whose reduced loops are OUTSIDE the output loops (back-propagation keeps the
  // forward loop order: `for b { for o { g[o] := g[o] + dz[b, o] } }`, or the fma form with two
  // factors).  A 32x32 block owns 32 consecutive outputs (threadIdx.x, coalesced) and splits the
  // flattened serial loop space over threadIdx.y; partial sums meet in shared memory and the
  // y == 0 row adds them to the node in a fixed order.
  bool ser_split_stage(Stage st, const Stmt& set) {
    if (set.kind != Stmt::Set) return false;
    const Tnode& t = code.prog.tn(set.tn);
    if (t.prec != Prec::Single && t.prec != Prec::Double) return false;
    int64_t ser_total = 1;
    for (auto& d : st.ser) ser_total *= d.extent();
    if (ser_total < 256) return false;
    // the written position must not move with a serial loop (an affine output position
    // `stride * o + k` of a convolution's input gradient does): then this is no reduction
    for (auto& d : st.ser)
      for (auto& ix : set.idcs)
        if (ix.uses(d.sym)) return false;
    const Scalar& v = *set.value;
    auto is_self = [&](const Scalar& e) {
      if (e.kind != Scalar::Get || e.tn != set.tn || e.idcs.size() != set.idcs.size()) return false;
      for (size_t i = 0; i < e.idcs.size(); ++i)
        if (e.idcs[i].kind != set.idcs[i].kind || e.idcs[i].sym != set.idcs[i].sym || e.idcs[i].fixed != set.idcs[i].fixed ||
            e.idcs[i].terms != set.idcs[i].terms)
          return false;
      return true;
    };
    auto reads_node = [&](const Scalar& e) {
      bool m = false;
      walk_scalar(e, [&](const Scalar& x) {
        if ((x.kind == Scalar::Get || x.kind == Scalar::GetDyn) && x.tn == set.tn) m = true;
        if (x.kind == Scalar::LocalScope) m = true;  // keep this path to plain terms
      }, [](const Stmt&) {});
      return m;
    };
    const Scalar *fa = nullptr, *fb = nullptr, *term = nullptr;
    if (v.kind == Scalar::Tern && v.op == "fma" && is_self(*v.args[2].s)) {
      fa = v.args[0].s.get();
      fb = v.args[1].s.get();
      if (reads_node(*fa) || reads_node(*fb)) return false;
    } else if (v.kind == Scalar::Bin && v.op == "add") {
      if (is_self(*v.args[0].s)) term = v.args[1].s.get();
      else if (is_self(*v.args[1].s)) term = v.args[0].s.get();
      if (!term || reads_node(*term)) return false;
    } else {
      return false;
    }
    Emitter em(code.prog);
    em.large_models = opt.large_models;
    // Pairs: a thread owns two neighbouring outputs along the innermost output loop when that loop
    // runs along the last axis of the fp32 node; the factors are then read as 4- and 8-byte words.
    bool pairs = false;
    if (pairs_here() && t.prec == Prec::Single && !st.par.empty() && !set.idcs.empty()) {
      const LoopDim& p = st.par.back();
      bool ok = p.from == 0 && p.extent() % 2 == 0 && set.idcs.back().kind == Index::Iter && set.idcs.back().sym == p.sym &&
                t.dims.back() % 2 == 0;
      for (size_t a = 0; ok && a + 1 < set.idcs.size(); ++a)
        if (set.idcs[a].uses(p.sym)) ok = false;
      if (ok && (term ? em.pair_supported(*term) : em.pair_supported(*fa) && em.pair_supported(*fb))) {
        pairs = true;
        em.pair = true;
        em.pair_sym = p.sym;
        em.pair_vector_loads = true;
      }
    }
    const std::string T = pairs ? "b200_f2" : Emitter::ctype(t.prec);
    const std::string zero = pairs ? "b200_f2{0.0f, 0.0f}" : "0";
    std::string step;
    if (pairs) {
      std::string pre;
      if (term) {
        const std::string v = em.pair_scalar(t.prec, *term, pre);
        step = "{\n" + pre + "          b200_acc = b200_f2{b200_acc.x + " + v + ".x, b200_acc.y + " + v + ".y};\n          }";
      } else {
        const std::string a = em.pair_scalar(t.prec, *fa, pre), b = em.pair_scalar(t.prec, *fb, pre);
        step = "{\n" + pre + "          b200_acc = b200_f2{fmaf(" + a + ".x, " + b + ".x, b200_acc.x), fmaf(" + a + ".y, " + b +
               ".y, b200_acc.y)};\n          }";
      }
      st.min_align = 8;
    } else if (term) {
      Emitter::Res r = em.scalar(t.prec, *term);
      if (!r.defs.empty()) return false;
      step = "b200_acc = b200_acc + " + r.expr + ";";
    } else {
      Emitter::Res ra = em.scalar(t.prec, *fa), rb = em.scalar(t.prec, *fb);
      if (!ra.defs.empty() || !rb.defs.empty()) return false;
      step = std::string("b200_acc = ") + (t.prec == Prec::Double ? "fma(" : "fmaf(") + ra.expr + ", " + rb.expr + ", b200_acc);";
    }
    em.used_nodes.insert(set.tn);
    for (auto& d : st.par) if (d.from != 0) return false;
    for (auto& d : st.ser) if (d.from != 0) return false;
    // Register tiling: a short outermost output loop (the 10 classes of `dW[o, i] += dz[b, o] * h[b, i]`)
    // stays inside the thread, which then reads the other factor once for all of its values.
    const bool tiled = !term && st.par.size() >= 2 && st.par[0].extent() <= 16;
    const int64_t e0 = tiled ? st.par[0].extent() : 1;
    const size_t first_par = tiled ? 1 : 0;
    const int64_t outputs = st.total / e0 / (pairs ? 2 : 1);   // output elements (or pairs) spread over threadIdx.x
    std::string decomp, sdecomp;
    {
      std::string rem = "b200_g";
      for (size_t i = st.par.size(); i-- > first_par;) {
        const LoopDim& d = st.par[i];
        const bool pair_dim = pairs && i + 1 == st.par.size();
        std::string ext = std::to_string(pair_dim ? d.extent() / 2 : d.extent()) + "ull";
        decomp += "      const unsigned int " + d.sym + " = " + (pair_dim ? "2u * " : "") + "(unsigned int)" +
                  (i == first_par ? rem : "(" + rem + " % " + ext + ")") + ";\n";
        if (i != first_par) {
          decomp += "      const unsigned long long b200_r" + std::to_string(i) + " = " + rem + " / " + ext + ";\n";
          rem = "b200_r" + std::to_string(i);
        }
      }
      rem = "b200_l";
      for (size_t i = st.ser.size(); i-- > 0;) {
        const LoopDim& d = st.ser[i];
        std::string ext = std::to_string(d.extent()) + "ull";
        sdecomp += "        const unsigned int " + d.sym + " = (unsigned int)" + (i == 0 ? rem : "(" + rem + " % " + ext + ")") + ";\n";
        if (i != 0) {
          sdecomp += "        const unsigned long long b200_q" + std::to_string(i) + " = " + rem + " / " + ext + ";\n";
          rem = "b200_q" + std::to_string(i);
        }
      }
    }
    const std::string off = em.offset(set.idcs, t.dims);
    std::string text = decomp + sdecomp + step + off;
    std::string statics = static_prologue(text, em, 2);
    // Few output groups leave most SMs idle: the serial loop space is then also cut into Z slices,
    // one block per (group, slice), and the slices meet in the output through atomic adds (their
    // order is not fixed; the node is fp32 or fp64 and already holds the value being added to).
    const int64_t groups = (outputs + 31) / 32;
    int64_t Z = 1;
    if (groups < 2 * 148) Z = std::max<int64_t>(1, std::min<int64_t>((4 * 148 + groups - 1) / groups, ser_total / 256));
    st.block = 32;
    st.block_y = 32;
    st.coop = 32;  // 32 threads per output element
    st.grid_override = (int)std::min<int64_t>(groups * Z, 148 * 8);
    std::set<int> written = {set.tn};
    const std::string o_sym = tiled ? st.par[0].sym : std::string();
    const std::string E0 = std::to_string(e0);
    std::ostringstream k;
    k << "extern \"C\" __global__ void __launch_bounds__(1024) " << st.kernel << "(";
    emit_params(k, st, em, written);
    k << ") {\n" << kGridEntry << statics << "  __shared__ " << T << " b200_part[32][33];\n"
      << "  for (unsigned long long b200_u = blockIdx.x; b200_u < " << groups * Z << "ull; b200_u += gridDim.x) {\n"
      << "    const unsigned long long b200_g = (b200_u % " << groups << "ull) * 32ull + threadIdx.x, b200_z = b200_u / " << groups << "ull;\n"
      << "    const unsigned long long b200_l0 = b200_z * " << ser_total << "ull / " << Z << "ull, b200_l1 = (b200_z + 1ull) * "
      << ser_total << "ull / " << Z << "ull;\n"
      << "    const bool b200_ok = b200_g < " << outputs << "ull;\n";
    if (tiled) k << "    " << T << " b200_accs[" << E0 << "];\n#pragma unroll\n    for (int b200_o = 0; b200_o < " << E0 << "; ++b200_o) b200_accs[b200_o] = " << zero << ";\n";
    else k << "    " << T << " b200_acc = " << zero << ";\n";
    k << "    if (b200_ok) {\n" << decomp
      << "#pragma unroll 4\n      for (unsigned long long b200_l = b200_l0 + threadIdx.y; b200_l < b200_l1; b200_l += 32ull) {\n" << sdecomp;
    if (tiled)
      k << "#pragma unroll\n        for (unsigned int " << o_sym << " = 0; " << o_sym << " < " << E0 << "u; ++" << o_sym << ") {\n"
        << "          " << T << " b200_acc = b200_accs[" << o_sym << "];\n          " << step << "\n          b200_accs[" << o_sym
        << "] = b200_acc;\n        }\n";
    else
      k << "        " << step << "\n";
    k << "      }\n    }\n";
    // combine the 32 slices of threadIdx.y, one output value (of the tiled loop) at a time
    if (tiled) k << "#pragma unroll\n    for (unsigned int " << o_sym << " = 0; " << o_sym << " < " << E0 << "u; ++" << o_sym << ") {\n      const "
                 << T << " b200_acc = b200_accs[" << o_sym << "];\n";
    else k << "    {\n";
    k << "      b200_part[threadIdx.y][threadIdx.x] = b200_acc;\n      __syncthreads();\n"
      << "      if (threadIdx.y == 0 && b200_ok) {\n" << decomp << "        " << T << " b200_s = " << zero << ";\n";
    if (pairs) {
      k << "        for (int b200_y = 0; b200_y < 32; ++b200_y) { b200_s.x += b200_part[b200_y][threadIdx.x].x; b200_s.y += b200_part[b200_y][threadIdx.x].y; }\n";
      if (Z > 1) k << "        atomicAdd(&" << t.ident << "[" << off << "], b200_s.x);\n        atomicAdd(&" << t.ident << "[(" << off << ") + 1], b200_s.y);\n";
      else k << "        " << t.ident << "[" << off << "] = " << t.ident << "[" << off << "] + b200_s.x;\n        " << t.ident << "[(" << off
             << ") + 1] = " << t.ident << "[(" << off << ") + 1] + b200_s.y;\n";
    } else {
      k << "        for (int b200_y = 0; b200_y < 32; ++b200_y) b200_s += b200_part[b200_y][threadIdx.x];\n";
      if (Z > 1) k << "        atomicAdd(&" << t.ident << "[" << off << "], b200_s);\n";
      else k << "        " << t.ident << "[" << off << "] = " << t.ident << "[" << off << "] + b200_s;\n";
    }
    k << "      }\n      __syncthreads();\n    }\n  }\n}\n\n";
    src << k.str();
    st.note = "par=" + std::to_string(st.par.size()) + " ser=" + std::to_string(st.ser.size()) + " serial loops split over a 32x32 block" +
              (Z > 1 ? ", " + std::to_string(Z) + " slices per output group (atomic adds)" : std::string()) +
              (tiled ? ", outer loop of " + E0 + " kept in registers" : std::string()) + (pairs ? ", pairs" : std::string());
    st.writes = {set.tn};
    code.stages.push_back(st);
    return true;
  }

  // Does `set` write every element of its node exactly once over `loops` (each axis a distinct
  // loop symbol running over the whole axis, or a fixed 0 on an axis of extent 1)?
  bool covers_node(const Stmt& set, const std::vector<LoopDim>& loops) {
    const Tnode& t = code.prog.tn(set.tn);
    if (set.kind != Stmt::Set || set.vec_len > 0 || set.idcs.size() != t.dims.size()) return false;
    std::set<std::string> seen;
    for (size_t a = 0; a < set.idcs.size(); ++a) {
      const Index& ix = set.idcs[a];
      if (ix.kind == Index::Fixed) {
        if (ix.fixed != 0 || t.dims[a] != 1) return false;
        continue;
      }
      if (ix.kind != Index::Iter || !seen.insert(ix.sym).second) return false;
      bool found = false;
      for (auto& d : loops)
        if (d.sym == ix.sym && d.from == 0 && d.extent() == t.dims[a]) found = true;
      if (!found) return false;
    }
    return true;
  }

  // `lhs_zero`: the node the body assigns is known to be all zero when the stage starts.
  // Returns true when the stage made an earlier zero_out of that node unnecessary.
  bool generic_stage(const std::vector<LoopDim>& nest, const StmtP& body, bool lhs_zero = false) {
    bool zero_out_dead = false;
    Stage st;
    st.kind = Stage::Generic;
    st.kernel = kernel_name();
    // which loops are independent
    std::vector<bool> par(nest.size(), false);
    for (size_t i = 0; i < nest.size(); ++i) par[i] = nest[i].extent() > 0 && parallel_safe(nest[i].sym, *body);
    for (size_t i = 0; i < nest.size(); ++i) (par[i] ? st.par : st.ser).push_back(nest[i]);
    st.total = 1;
    for (auto& d : st.par) st.total *= d.extent();
    for (auto& d : nest)
      if (d.extent() <= 0) st.total = 0;

    Emitter em(code.prog);
    em.large_models = opt.large_models;

    // Scatter accumulation: `t[.., c * o + k, ..] := t[same] + term` where the written position
    // moves with loops that therefore cannot run in parallel (the input gradient of a
    // convolution).  Those loops are spread over threads all the same: a thread sums over the
    // loops that do not move the position and adds its partial sum with one atomic add.
    bool scatter = false;
    if (opt.enable_coop && !st.ser.empty() && st.total > 0 && body->kind == Stmt::Set && body->vec_len == 0 &&
        accumulates_into_self(*body)) {
      const Tnode& t = code.prog.tn(body->tn);
      std::vector<LoopDim> spread, kept;
      for (auto& d : nest) {
        bool in_par = false, moves = false;
        for (auto& q : st.par) in_par = in_par || q.sym == d.sym;
        for (auto& ix : body->idcs) moves = moves || ix.uses(d.sym);
        (in_par || moves ? spread : kept).push_back(d);
      }
      int64_t total = 1;
      for (auto& d : spread) total *= d.extent();
      if ((t.prec == Prec::Single || t.prec == Prec::Double) && t.mode != Mode::Virtual && spread.size() > st.par.size() &&
          total >= 4096) {
        scatter = true;
        st.par = spread;
        st.ser = kept;
        st.total = total;
      }
    }

    if (!scatter && !st.ser.empty() && st.total > 0 && opt.enable_coop && ser_split_stage(st, *body)) return false;

    CoopInfo ci;
    if (st.ser.empty() && st.total > 0) ci = find_coop(*body, st.total);
    if (ci.grid_blocks > 0) {
      --next_kernel;  // the name reserved above is re-issued to the first pass
      grid_reduce_stage(body, ci);
      return false;
    }
    std::set<int> written;
    walk_stmt(*body, [](const Scalar&) {}, [&](const Stmt& s) {
      if (s.kind == Stmt::Set || s.kind == Stmt::ZeroOut) written.insert(s.tn);
    });

    // Pairs.  When the stage is one assignment whose innermost parallel loop runs along the last
    // axis of the written node, and everything in it is fp32, bf16 or half, a thread takes TWO
    // neighbouring iterations of that loop: 4- and 8-byte accesses, packed 16-bit arithmetic.
    bool pairs = false;
    if (pairs_here() && !scatter && ci.sym.empty() && body->kind == Stmt::Set && body->vec_len == 0 && !st.par.empty() && st.total > 0) {
      const Stmt& set = *body;
      const Tnode& t = code.prog.tn(set.tn);
      const LoopDim& p = st.par.back();
      bool ok = p.from == 0 && p.extent() % 2 == 0 && Emitter::pair_prec(t.prec) && t.mode != Mode::Virtual && !set.idcs.empty() &&
                set.idcs.back().kind == Index::Iter && set.idcs.back().sym == p.sym && t.dims.back() % 2 == 0;
      for (size_t a = 0; ok && a + 1 < set.idcs.size(); ++a)
        if (set.idcs[a].uses(p.sym)) ok = false;
      // reads of the written node only at the written position (they become the promoted register)
      walk_scalar(*set.value, [&](const Scalar& e) {
        if (e.kind == Scalar::GetDyn && e.tn == set.tn) ok = false;
      }, [](const Stmt&) {});
      if (ok && em.pair_supported(*set.value)) {
        pairs = true;
        em.pair = true;
        em.pair_sym = p.sym;
        em.pair_vector_loads = true;
      }
    }
    // Accumulator promotion: `t[p] := f(t[p], ...)` under serial loops that do not move p keeps
    // t[p] in a register across those loops (one load, or none when the node is known to be zero,
    // and one store) instead of a read-modify-write of memory per iteration.
    std::string before, after;
    if (scatter) {
      const Stmt& set = *body;
      const Tnode& t = code.prog.tn(set.tn);
      em.used_nodes.insert(set.tn);
      before = std::string("    ") + Emitter::ctype(t.prec) + " b200_self = 0;\n";
      after = "    atomicAdd(&" + t.ident + "[" + em.offset(set.idcs, t.dims) + "], b200_self);\n";
      em.forwarded[set.tn] = {set.idcs, "b200_self"};
      em.set_redirect[set.tn] = {set.idcs, "b200_self"};
    } else if (ci.sym.empty() && (pairs || !st.ser.empty()) && body->kind == Stmt::Set && body->vec_len == 0) {
      const Stmt& set = *body;
      const Tnode& t = code.prog.tn(set.tn);
      bool ok = t.mode != Mode::Virtual && t.prec != Prec::Uint4x32;
      for (auto& ix : set.idcs)
        for (auto& d : st.ser)
          if (ix.uses(d.sym)) ok = false;
      int self_reads = 0;
      walk_scalar(*set.value, [&](const Scalar& e) {
        if (e.kind == Scalar::LocalScope) ok = false;
        if ((e.kind == Scalar::Get || e.kind == Scalar::GetDyn) && e.tn == set.tn) {
          bool same = e.kind == Scalar::Get && e.idcs.size() == set.idcs.size();
          for (size_t i = 0; same && i < e.idcs.size(); ++i)
            if (e.idcs[i].kind != set.idcs[i].kind || e.idcs[i].sym != set.idcs[i].sym || e.idcs[i].fixed != set.idcs[i].fixed ||
                e.idcs[i].terms != set.idcs[i].terms)
              same = false;
          if (same) ++self_reads; else ok = false;
        }
      }, [](const Stmt&) {});
      if (ok && self_reads > 0) {
        const std::string off = em.offset(set.idcs, t.dims);
        const std::string lv = t.ident + "[" + off + "]";
        em.used_nodes.insert(set.tn);
        if (pairs) {
          const std::string PT = Emitter::pair_type(t.prec);
          const std::string at = "(" + t.ident + " + " + off + ")";
          before = "    " + PT + " b200_self = " +
                   (lhs_zero ? (t.prec == Prec::Single ? std::string("b200_f2{0.0f, 0.0f}") : std::string("0u")) : "*(const " + PT + "*)" + at) + ";\n";
          after = "    *(" + PT + "*)" + at + " = b200_self;\n";
        } else {
          before = std::string("    ") + Emitter::rtype(t.prec) + " b200_self = " +
                   (lhs_zero ? em.constant(0.0, t.prec) : Emitter::load_wrap(t.prec, lv)) + ";\n";
          after = "    " + lv + " = " + Emitter::store_wrap(t.prec, "b200_self") + ";\n";
        }
        em.forwarded[set.tn] = {set.idcs, "b200_self"};
        em.set_redirect[set.tn] = {set.idcs, "b200_self"};
        zero_out_dead = lhs_zero && covers_node(set, st.par);
      }
    }
    if (pairs && before.empty()) {
      // without promotion a read of the written node would be a plain (unpaired) memory access
      bool self = false;
      walk_scalar(*body->value, [&](const Scalar& e) {
        if ((e.kind == Scalar::Get || e.kind == Scalar::GetDyn) && e.tn == body->tn) self = true;
      }, [](const Stmt&) {});
      if (self) {
        pairs = false;
        em.pair = false;
        em.pair_vector_loads = false;
      }
    }
    if (pairs) {
      st.total /= 2;      // one thread per pair
      st.min_align = 8;   // pairs are read and written as 4- and 8-byte words
    }
    // Small tables read over and over.  A read-only node of at most 32 KB that the stage reads inside
    // a reduction or serial loop, many times per element (the 512 x 27 embedding table of a one-hot
    // contraction with K = 27: rows of 54 bytes, no tensor-map can describe them) is copied into
    // shared memory once per block; the strided reads then hit shared-memory banks instead of L1
    // sectors.  Such a stage keeps its own kernel (few blocks, each looping over many elements).
    std::vector<int> staged;
    if (opt.enable_coop && !scatter && !pairs && ci.sym.empty() && body->kind == Stmt::Set && st.total > 0) {
      int64_t work = st.total;
      for (auto& d : st.ser) work *= std::max<int64_t>(1, d.extent());
      std::set<std::string> inner_syms;
      for (auto& d : st.ser) inner_syms.insert(d.sym);
      walk_stmt(*body, [](const Scalar&) {}, [&](const Stmt& x) { if (x.kind == Stmt::For) inner_syms.insert(x.index); });
      int64_t inner_iters = 1;
      walk_stmt(*body, [](const Scalar&) {}, [&](const Stmt& x) { if (x.kind == Stmt::For) inner_iters *= std::max<int64_t>(1, x.to - x.from + 1); });
      std::set<int> cand;
      size_t bytes = 0;
      walk_scalar(*body->value, [&](const Scalar& e) {
        if (e.kind != Scalar::Get) return;
        const Tnode& t = code.prog.tn(e.tn);
        if (!t.read_only || t.mode == Mode::Virtual || written.count(e.tn) || t.bytes() > 32768 || t.prec == Prec::Uint4x32) return;
        bool in_loop = false;
        for (auto& ix : e.idcs)
          for (auto& sy : inner_syms) in_loop = in_loop || ix.uses(sy);
        if (in_loop && work * inner_iters >= 256 * t.num_elems()) cand.insert(e.tn);
      }, [](const Stmt&) {});
      // first the nodes indexed by the innermost parallel loop: their reads differ from thread to
      // thread (a read that is the same for a whole warp is one broadcast access anyway)
      std::vector<int> order(cand.begin(), cand.end());
      auto strided = [&](int tn) {
        bool u = false;
        walk_scalar(*body->value, [&](const Scalar& e) {
          if (e.kind == Scalar::Get && e.tn == tn && !st.par.empty())
            for (auto& ix : e.idcs) u = u || ix.uses(st.par.back().sym);
        }, [](const Stmt&) {});
        return u;
      };
      std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return strided(a) > strided(b); });
      for (int tn : order) {
        if (bytes + (size_t)code.prog.tn(tn).bytes() > 40960) continue;
        bytes += (size_t)code.prog.tn(tn).bytes();
        staged.push_back(tn);
        em.node_alias[tn] = "b200_sm_" + code.prog.tn(tn).ident;
      }
      if (!staged.empty() && inner_iters < 8) {   // nothing is re-read often enough
        staged.clear();
        em.node_alias.clear();
      }
    }
    std::string inner;
    int ind = 4 + 2 * (int)st.ser.size();
    if (!ci.sym.empty()) {
      st.coop = ci.width;
      if (ci.width > 32) st.block = ci.width;
      inner = coop_body(em, *body, ci, ind);
    } else {
      inner = em.stmt(*body, ind);
    }
    // serial loops wrap the body in their original order
    std::string open, close;
    int k = 4;
    for (auto& d : st.ser) {
      open += std::string((size_t)k, ' ') + "for (unsigned int " + d.sym + " = " + std::to_string(d.from) + "; " + d.sym +
              " <= " + std::to_string(d.to) + "; ++" + d.sym + ") {\n";
      k += 2;
    }
    for (size_t i = st.ser.size(); i-- > 0;) {
      k -= 2;
      close += std::string((size_t)k, ' ') + "}\n";
    }
    std::string body_text = before + open + inner + close + after;

    // index decomposition: the innermost parallel loop varies fastest across threads
    // (in 32-bit arithmetic when the flattened count fits: 64-bit divisions by constants cost
    // several times as many instructions, and pointwise kernels are made of little else)
    std::string decomp;
    {
      const bool narrow = st.total < (1ll << 31);
      const std::string IT = narrow ? "unsigned int" : "unsigned long long", SUF = narrow ? "u" : "ull";
      std::string rem = "b200_g";
      if (narrow && st.par.size() > 1) {
        decomp += "    const unsigned int b200_g32 = (unsigned int)b200_g;\n";
        rem = "b200_g32";
      }
      for (size_t i = st.par.size(); i-- > 0;) {
        const LoopDim& d = st.par[i];
        const bool pair_dim = pairs && i + 1 == st.par.size();   // iterations of this loop are taken two at a time
        std::string ext = std::to_string(pair_dim ? d.extent() / 2 : d.extent()) + SUF;
        std::string val = i == 0 ? rem : "(" + rem + " % " + ext + ")";
        decomp += "    const unsigned int " + d.sym + " = " + (pair_dim ? "2u * " : "") + "(unsigned int)" + val +
                  (d.from ? " + " + std::to_string(d.from) : std::string()) + ";\n";
        if (i != 0) {
          std::string nr = "b200_r" + std::to_string(i);
          decomp += "    const " + IT + " " + nr + " = " + rem + " / " + ext + ";\n";
          rem = nr;
        }
      }
    }
    // the kernel text is assembled at the end of the routine (emit_kernels), when it is known
    // which neighbouring stages are small enough to share one launch
    Piece pc;
    pc.decomp = decomp;
    pc.body_text = body_text;
    pc.used = em.used_nodes;
    pc.written = written;
    pc.uses_merge = em.uses_merge;
    int64_t ser_work = 1;
    for (auto& d : st.ser) ser_work *= std::max<int64_t>(1, d.extent());
    pc.fusable = opt.enable_fuse && st.total > 0 && (st.coop == 0 || st.coop == 32) &&
                 st.total * std::max(1, st.coop) <= 16384 && ser_work <= 4096;
    if (scatter) pc.fusable = false;
    if (opt.enable_fuse && !scatter && st.coop == 0 && st.total > 0 && !st.par.empty() && st.par[0].from == 0 && !(pairs && st.par.size() == 1)) {
      pc.body = body;
      pc.row_sym = st.par[0].sym;
      pc.rows = st.par[0].extent();
      pc.per_row = st.total / pc.rows * ser_work;
    }
    if (!scatter) pc.any_body = body;
    if (!staged.empty()) {      // keeps a kernel of its own
      pc.staged = staged;
      pc.fusable = false;
      pc.body = nullptr;
      pc.any_body = nullptr;
      st.grid_override = 148 * 4;
      st.block = 512;
    }
    pc.par = st.par;
    pc.coop = st.coop;
    pc.pairs = pairs;
    pc.ser_work = ser_work;
    std::ostringstream note;
    note << "par=" << st.par.size() << " ser=" << st.ser.size()
         << (st.coop > 32 ? " block-per-element" : st.coop ? " warp-per-element" : "") << (pairs ? " pairs" : "")
         << (scatter ? " scatter accumulation (atomic adds)" : "") << (staged.empty() ? "" : " small table staged in shared memory");
    st.note = note.str();
    pieces[code.stages.size()] = pc;
    st.writes.assign(written.begin(), written.end());
    code.stages.push_back(st);
    return zero_out_dead;
  }

  // Text of one stand-alone generic kernel (grid-stride over the stage's parallel iterations).
  void emit_single(Stage& st, const Piece& pc) {
    Emitter em(code.prog);
    em.used_nodes = pc.used;
    em.uses_merge = pc.uses_merge;
    std::string statics = static_prologue(pc.body_text + pc.decomp, em, 2);
    std::ostringstream k_src;
    k_src << "extern \"C\" __global__ void __launch_bounds__(" << st.block << ") " << st.kernel << "(";
    emit_params(k_src, st, em, pc.written);
    k_src << ") {\n" << kGridEntry << statics;
    for (int tn : pc.staged) {
      const Tnode& t = code.prog.tn(tn);
      const std::string sm = "b200_sm_" + t.ident;
      k_src << "  __shared__ " << Emitter::ctype(t.prec) << " " << sm << "[" << t.num_elems() << "];\n"
            << "  for (unsigned int b200_i = threadIdx.x; b200_i < " << t.num_elems() << "u; b200_i += blockDim.x) " << sm
            << "[b200_i] = " << t.ident << "[b200_i];\n";
    }
    if (!pc.staged.empty()) k_src << "  __syncthreads();\n";
    if (st.coop > 32) {
      k_src << "  __shared__ double b200_red[32];\n";
      k_src << "  const unsigned int b200_t = threadIdx.x;\n";
      k_src << "  for (unsigned long long b200_g = blockIdx.x; b200_g < " << st.total << "ull; b200_g += gridDim.x) {\n";
    } else if (st.coop) {
      k_src << "  const unsigned int b200_t = threadIdx.x & 31u;\n";
      k_src << "  const unsigned long long b200_warp = ((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;\n";
      k_src << "  const unsigned long long b200_nwarps = ((unsigned long long)gridDim.x * blockDim.x) >> 5;\n";
      k_src << "  for (unsigned long long b200_g = b200_warp; b200_g < " << st.total << "ull; b200_g += b200_nwarps) {\n";
    } else {
      k_src << "  for (unsigned long long b200_g = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; b200_g < "
            << st.total << "ull; b200_g += (unsigned long long)gridDim.x * blockDim.x) {\n";
    }
    k_src << pc.decomp << pc.body_text << "  }\n}\n\n";
    src << k_src.str();
  }

  // Several small consecutive stages (and small zero_outs) as ONE kernel of a single
  // 1024-thread block: each stage strides its iterations over the block, __syncthreads()
  // separates the stages.  Launch latency, not work, dominates such routines (the 2-16-16-1
  // training step is ~30 stages of a few hundred iterations each).
  void merge_origins(Stage& f, const std::vector<size_t>& idx) {
    std::set<int> all;
    std::set<int> w;
    for (size_t i : idx) {
      all.insert(code.stages[i].origins.begin(), code.stages[i].origins.end());
      w.insert(code.stages[i].writes.begin(), code.stages[i].writes.end());
    }
    f.origins.assign(all.begin(), all.end());
    f.writes.assign(w.begin(), w.end());
  }

  Stage emit_fused(const std::vector<size_t>& idx) {
    Stage f;
    merge_origins(f, idx);
    f.kind = Stage::Generic;
    f.kernel = code.stages[idx.front()].kernel.empty() ? kernel_name() : code.stages[idx.front()].kernel;
    f.block = 1024;
    f.grid_override = 1;
    f.total = 1;
    Emitter em(code.prog);
    std::set<int> written;
    std::string text;
    for (size_t i : idx) {
      const Stage& st = code.stages[i];
      if (st.kind == Stage::Memset) {
        const Tnode& t = code.prog.tn(st.memset_tn);
        em.used_nodes.insert(t.id);
        written.insert(t.id);
        text += "  for (unsigned int b200_z = threadIdx.x; b200_z < " + std::to_string(t.num_elems()) +
                "u; b200_z += blockDim.x) " + t.ident + "[b200_z] = " + em.storage_zero(t.prec) + ";\n";
      } else {
        const Piece& pc = pieces[i];
        f.min_align = std::max(f.min_align, st.min_align);
        em.used_nodes.insert(pc.used.begin(), pc.used.end());
        written.insert(pc.written.begin(), pc.written.end());
        em.uses_merge |= pc.uses_merge;
        text += "  {\n";
        if (st.coop) {
          text += "  const unsigned int b200_t = threadIdx.x & 31u;\n";
          text += "  for (unsigned long long b200_g = threadIdx.x >> 5; b200_g < " + std::to_string(st.total) +
                  "ull; b200_g += blockDim.x >> 5) {\n";
        } else {
          text += "  for (unsigned long long b200_g = threadIdx.x; b200_g < " + std::to_string(st.total) +
                  "ull; b200_g += blockDim.x) {\n";
        }
        text += pc.decomp + pc.body_text + "  }\n  }\n";
      }
      text += "  __syncthreads();\n";
    }
    std::string statics = static_prologue(text, em, 2);
    std::ostringstream k_src;
    k_src << "extern \"C\" __global__ void __launch_bounds__(1024) " << f.kernel << "(";
    emit_params(k_src, f, em, written);
    k_src << ") {\n" << kGridEntry << statics << text << "}\n\n";
    src << k_src.str();
    f.note = "fused " + std::to_string(idx.size()) + " small stages in one block";
    return f;
  }

  // Warp-per-row fusion.  A run of stages that share their L outermost parallel loops ("the
  // row": (batch, position, head) of an attention softmax), some of which reduce over the rest of
  // the row with a warp per output element while others are pointwise along it, and which hand
  // data to one another only within a row, runs as ONE kernel: a warp takes a row and executes
  // the stages one after the other, its lanes striding over the row.  Row max, exponentials, row
  // sum and the division of a softmax are one launch; the row stays in L1 / L2 between them.
  bool rows_independent_prefix(const std::vector<size_t>& run, size_t L) {
    std::map<int, int> writers, users;
    for (size_t i : run) {
      const Piece& pc = pieces[i];
      for (int n : pc.written) writers[n]++;
      for (int n : pc.used) users[n]++;
    }
    std::map<std::pair<int, size_t>, int> axis;  // (shared node, prefix position) -> axis carrying that loop's symbol
    bool ok = true;
    for (size_t i : run) {
      const Piece& pc = pieces[i];
      auto check = [&](int tn, const Indices& idcs) {
        if (!writers.count(tn) || users[tn] < 2) return;
        for (size_t q = 0; q < L; ++q) {
          if (pc.par[q].extent() == 1) continue;   // a loop of one iteration separates nothing
          const std::string& sym = pc.par[q].sym;
          int a = -1;
          for (size_t k = 0; k < idcs.size(); ++k) {
            if (idcs[k].kind == Index::Iter && idcs[k].sym == sym && a < 0) a = (int)k;
            else if (idcs[k].uses(sym)) ok = false;
          }
          if (a < 0) { ok = false; return; }
          auto it = axis.find({tn, q});
          if (it == axis.end()) axis[{tn, q}] = a;
          else if (it->second != a) ok = false;
        }
      };
      walk_stmt(
          *pc.any_body,
          [&](const Scalar& e) {
            if (e.kind == Scalar::Get) check(e.tn, e.idcs);
            if (e.kind == Scalar::GetDyn && writers.count(e.tn) && users[e.tn] >= 2) ok = false;
          },
          [&](const Stmt& st) {
            if (st.kind == Stmt::Set) {
              if (st.vec_len > 0 && writers.count(st.tn) && users[st.tn] >= 2) ok = false;
              check(st.tn, st.idcs);
            }
            if (st.kind == Stmt::ZeroOut) ok = false;
          });
    }
    return ok;
  }

  // can stage i join a warp-per-row group whose rows are the first L parallel loops of `like`?
  bool warp_row_member(size_t i, size_t L, const Piece* like) {
    auto it = pieces.find(i);
    if (it == pieces.end() || !it->second.any_body) return false;
    const Piece& pc = it->second;
    if (pc.coop != 0 && pc.coop != 32) return false;
    if (pc.par.size() < L || (pc.coop == 32 && pc.par.size() != L)) return false;
    if (pc.pairs && pc.par.size() == L) return false;   // the pair loop must lie inside the row
    for (size_t q = 0; q < L; ++q) {
      if (pc.par[q].from != 0) return false;
      if (like && pc.par[q].extent() != like->par[q].extent()) return false;
    }
    return true;
  }

  Stage emit_warp_rows(const std::vector<size_t>& run, size_t L) {
    Stage f;
    merge_origins(f, run);
    f.kind = Stage::Generic;
    f.kernel = code.stages[run.front()].kernel;
    f.block = 256;
    int64_t rows = 1;
    for (size_t q = 0; q < L; ++q) rows *= pieces[run.front()].par[q].extent();
    f.total = rows;
    f.coop = 32;   // launch arithmetic: 32 threads per row
    Emitter em(code.prog);
    std::set<int> written;
    std::string text;
    for (size_t i : run) {
      const Stage& st = code.stages[i];
      const Piece& pc = pieces[i];
      f.min_align = std::max(f.min_align, st.min_align);
      em.used_nodes.insert(pc.used.begin(), pc.used.end());
      written.insert(pc.written.begin(), pc.written.end());
      em.uses_merge |= pc.uses_merge;
      if (pc.coop == 32) {
        text += "    {\n    const unsigned long long b200_g = b200_row;\n" + pc.decomp + pc.body_text + "    }\n";
      } else {
        const std::string inner = std::to_string(st.total / rows) + "ull";
        text += "    for (unsigned long long b200_g = b200_row * " + inner + " + b200_t; b200_g < (b200_row + 1ull) * " + inner +
                "; b200_g += 32ull) {\n" + pc.decomp + pc.body_text + "    }\n";
      }
      text += "    __syncwarp();\n";   // orders the row's stores before the next stage's loads
    }
    std::string statics = static_prologue(text, em, 2);
    std::ostringstream k_src;
    k_src << "extern \"C\" __global__ void __launch_bounds__(" << f.block << ") " << f.kernel << "(";
    emit_params(k_src, f, em, written);
    k_src << ") {\n" << kGridEntry << statics
          << "  const unsigned int b200_t = threadIdx.x & 31u;\n"
          << "  const unsigned long long b200_warp = ((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;\n"
          << "  const unsigned long long b200_nwarps = ((unsigned long long)gridDim.x * blockDim.x) >> 5;\n"
          << "  for (unsigned long long b200_row = b200_warp; b200_row < " << rows << "ull; b200_row += b200_nwarps) {\n"
          << text << "  }\n}\n\n";
    src << k_src.str();
    f.note = "row-fused " + std::to_string(run.size()) + " stages, one warp per row";
    return f;
  }

  // ---- register-resident rows.  The warp-per-row kernel above lets its stages meet through memory:
  // every stage strides the row again, decomposes indices again and reloads from L1 what the
  // stage before stored.  When every stage is one assignment and touches the shared nodes only at
  // "the row's element t" (t on the node's last, contiguous axis) or at one value per row, a lane
  // instead owns R / 32 CONSECUTIVE elements of the row for the whole kernel: inputs are loaded
  // once with 16-byte accesses into register arrays, reductions run over the lane's registers
  // and one shuffle tree, every produced row is kept in registers for the stages after it and
  // stored once, with 16-byte accesses.  (Softmax over 256 keys: the scores are read once, the
  // exponentials and the weights written once each; layer norm over 512 features likewise.)
  static StmtP rename_stmt(const StmtP& s, const std::map<std::string, std::string>& ren) {
    auto c = std::make_shared<Stmt>(*s);
    rename_idcs(c->idcs, ren);
    auto it = ren.find(c->index);
    if (it != ren.end()) c->index = it->second;
    for (auto& x : c->items) x = rename_stmt(x, ren);
    if (c->body) c->body = rename_stmt(c->body, ren);
    if (c->value) c->value = rename_scalar(c->value, ren);
    return c;
  }
  static void rename_idcs(Indices& idcs, const std::map<std::string, std::string>& ren) {
    for (auto& ix : idcs) {
      if (ix.kind == Index::Iter) {
        auto it = ren.find(ix.sym);
        if (it != ren.end()) ix.sym = it->second;
      } else if (ix.kind == Index::Affine) {
        for (auto& t : ix.terms) {
          auto it = ren.find(t.second);
          if (it != ren.end()) t.second = it->second;
        }
      }
    }
  }
  static ScalarP rename_scalar(const ScalarP& e, const std::map<std::string, std::string>& ren) {
    auto c = std::make_shared<Scalar>(*e);
    rename_idcs(c->idcs, ren);
    {
      Indices one = {c->idx};
      rename_idcs(one, ren);
      c->idx = one[0];
    }
    if (c->body) c->body = rename_stmt(c->body, ren);
    for (auto& a : c->args) a.s = rename_scalar(a.s, ren);
    return c;
  }

  struct RegRowStage {
    StmtP set;                       // the assignment, row symbols renamed to the canonical ones
    bool coop = false;
    std::string t_sym;               // pointwise: the stage's element loop
    std::vector<std::pair<int, std::string>> scopes;   // coop: (scope id, combine op)
    std::vector<std::string> scope_syms;               // coop: each scope's element loop
  };

  bool emit_warp_rows_reg(const std::vector<size_t>& run, size_t L, Stage* out) {
    if (!opt.enable_pairs) return false;
    const Piece& first = pieces[run.front()];
    std::vector<std::string> canon;
    int64_t rows = 1;
    for (size_t q = 0; q < L; ++q) {
      canon.push_back("b200_r" + std::to_string(q) + "_" + first.par[q].sym);
      rows *= first.par[q].extent();
    }
    int64_t R = -1;
    std::vector<RegRowStage> stages;
    for (size_t i : run) {
      if (opt.no_pairs_at.count(code.stages[i].origins.empty() ? -1 : code.stages[i].origins[0])) return false;
      const Piece& pc = pieces[i];
      if (!pc.any_body || pc.any_body->kind != Stmt::Set || pc.any_body->vec_len > 0) return false;
      RegRowStage st;
      std::map<std::string, std::string> ren;
      for (size_t q = 0; q < L; ++q) ren[pc.par[q].sym] = canon[q];
      st.set = rename_stmt(pc.any_body, ren);
      if (pc.coop == 32) {
        st.coop = true;
        if (pc.par.size() != L) return false;
        CoopInfo ci = find_coop(*pc.any_body, 1 << 20);
        if (ci.sym.empty() || ci.width != 32) return false;
        st.scopes = ci.scopes;
        // every scope: [v := neutral;] for k = 0 .. R-1 { v := v op term }
        bool ok = true;
        std::function<void(const Scalar&)> rec = [&](const Scalar& e) {
          if (e.kind == Scalar::LocalScope) {
            const Stmt* b = e.body.get();
            if (b->kind == Stmt::Seq) b = b->items[1].get();
            if (b->kind != Stmt::For || b->from != 0 || b->body->kind == Stmt::For) { ok = false; return; }
            const int64_t ext = b->to + 1;
            if (R < 0) R = ext;
            if (ext != R) ok = false;
            st.scope_syms.push_back(b->index);
            return;
          }
          for (auto& a : e.args) rec(*a.s);
        };
        rec(*st.set->value);
        if (!ok || st.scope_syms.size() != st.scopes.size()) return false;
      } else {
        if (pc.coop != 0 || pc.par.size() != L + 1 || pc.ser_work != 1) return false;
        const LoopDim& t = pc.par[L];
        if (t.from != 0) return false;
        if (R < 0) R = t.extent();
        if (t.extent() != R) return false;
        st.t_sym = t.sym;
        bool scopes = false;
        walk_scalar(*st.set->value, [&](const Scalar& e) { if (e.kind == Scalar::LocalScope || e.kind == Scalar::GetLocal) scopes = true; },
                    [](const Stmt&) {});
        if (scopes) return false;
      }
      stages.push_back(st);
    }
    if (R < 64 || R % 32 != 0) return false;
    const int EPL = (int)(R / 32);
    if (EPL != 2 && EPL != 4 && EPL != 8 && EPL != 16) return false;

    // ---- classify every access
    struct RowNode { Indices idcs; Prec prec; bool loaded = false, produced = false; int writer = -1; };
    std::map<int, RowNode> rownodes;        // nodes touched at (row.., t)
    std::map<int, std::pair<Indices, int>> scalars;   // nodes written once per row: (indices, writing stage)
    auto uses_any = [&](const Indices& idcs, const std::set<std::string>& syms) {
      for (auto& ix : idcs)
        for (auto& sy : syms)
          if (ix.uses(sy)) return true;
      return false;
    };
    bool ok = true;
    std::set<int> written_nodes;
    for (size_t k = 0; k < stages.size(); ++k) {
      const RegRowStage& st = stages[k];
      std::set<std::string> tsyms(st.scope_syms.begin(), st.scope_syms.end());
      if (!st.t_sym.empty()) tsyms.insert(st.t_sym);
      auto row_position = [&](int tn, const Indices& idcs) {
        // last index is exactly an element symbol, on a last axis of extent R; no other use of it
        const Tnode& t = code.prog.tn(tn);
        if (idcs.empty() || idcs.size() != t.dims.size()) return false;
        const Index& last = idcs.back();
        if (last.kind != Index::Iter || !tsyms.count(last.sym) || t.dims.back() != R) return false;
        Indices rest(idcs.begin(), idcs.end() - 1);
        if (uses_any(rest, tsyms)) return false;
        for (auto& ix : rest)
          if (ix.kind != Index::Iter && ix.kind != Index::Fixed) return false;
        return t.prec == Prec::Single || t.prec == Prec::Bfloat16 || t.prec == Prec::Half;
      };
      auto note_row = [&](int tn, const Indices& idcs, bool write) {
        Indices key(idcs.begin(), idcs.end() - 1);
        auto it = rownodes.find(tn);
        if (it == rownodes.end()) {
          RowNode rn;
          rn.idcs = key;
          rn.prec = code.prog.tn(tn).prec;
          it = rownodes.emplace(tn, rn).first;
        } else {
          if (it->second.idcs.size() != key.size()) { ok = false; return; }
          for (size_t a = 0; a < key.size(); ++a)
            if (key[a].kind != it->second.idcs[a].kind || key[a].sym != it->second.idcs[a].sym || key[a].fixed != it->second.idcs[a].fixed) ok = false;
        }
        if (write) {
          if (it->second.produced || it->second.loaded) ok = false;    // written twice, or read before it is written
          it->second.produced = true;
          it->second.writer = (int)k;
        } else if (!it->second.produced) {
          it->second.loaded = true;
        }
      };
      // reads
      walk_scalar(*st.set->value, [&](const Scalar& e) {
        if (e.kind == Scalar::GetDyn || e.kind == Scalar::GetMerge) { ok = false; return; }
        if (e.kind != Scalar::Get) return;
        if (uses_any(e.idcs, tsyms)) {
          if (!row_position(e.tn, e.idcs)) {
            // an element-dependent read of a node this kernel does not write may stay a plain load
            if (written_nodes.count(e.tn)) ok = false;
            bool later = false;
            for (size_t k2 = k; k2 < stages.size(); ++k2) later = later || stages[k2].set->tn == e.tn;
            if (later) ok = false;
            return;
          }
          note_row(e.tn, e.idcs, false);
        } else if (written_nodes.count(e.tn)) {
          auto it = scalars.find(e.tn);
          if (it == scalars.end()) { ok = false; return; }
          if (e.idcs.size() != it->second.first.size()) { ok = false; return; }
          for (size_t a = 0; a < e.idcs.size(); ++a)
            if (e.idcs[a].kind != it->second.first[a].kind || e.idcs[a].sym != it->second.first[a].sym ||
                e.idcs[a].fixed != it->second.first[a].fixed)
              ok = false;
        }
      }, [](const Stmt&) {});
      // the write
      const Stmt& set = *st.set;
      if (st.coop) {
        if (uses_any(set.idcs, tsyms) || written_nodes.count(set.tn) || rownodes.count(set.tn)) ok = false;
        for (auto& ix : set.idcs)
          if (ix.kind != Index::Iter && ix.kind != Index::Fixed) ok = false;
        scalars[set.tn] = {set.idcs, (int)k};
      } else {
        if (!row_position(set.tn, set.idcs) || written_nodes.count(set.tn)) ok = false;
        else note_row(set.tn, set.idcs, true);
      }
      written_nodes.insert(set.tn);
      if (!ok) return false;
    }
    // a node read at other positions by a LATER plain load after being written here was refused above;
    // a row node that is both loaded and produced was refused as well

    // ---- emit
    Stage f;
    f.kind = Stage::Generic;
    f.kernel = code.stages[run.front()].kernel;
    f.block = 256;
    f.total = rows;
    f.coop = 32;
    merge_origins(f, run);
    Emitter em(code.prog);
    em.large_models = opt.large_models;
    em.unroll_loops = true;
    std::set<int> written;
    for (size_t i : run) {
      const Piece& pc = pieces[i];
      em.used_nodes.insert(pc.used.begin(), pc.used.end());
      written.insert(pc.written.begin(), pc.written.end());
      em.uses_merge |= pc.uses_merge;
    }
    int max_bytes = 4;
    auto reg = [](int tn) { return "b200_row" + std::to_string(tn); };
    // Which elements of a row a lane owns.  Four at a time, dealt round the warp (element
    // (k * 32 + lane) * 4 + j in register 4 k + j) when the lane's share is a multiple of four: every
    // access of the warp then covers one contiguous stretch of the row.  A share of two elements stays
    // consecutive (lane * 2 + e).
    const bool dealt = EPL % 4 == 0;
    const std::string own = dealt ? "(((b200_e >> 2) * 32u + b200_t) * 4u + (b200_e & 3u))" : "(b200_t0 + b200_e)";
    auto row_ptr = [&](int tn, const RowNode& rn) {
      const Tnode& t = code.prog.tn(tn);
      Indices at = rn.idcs;
      Index zero;
      at.push_back(zero);
      return t.ident + " + (" + em.offset(at, t.dims) + ")" + (dealt ? "" : " + b200_t0");
    };
    auto ld = [&](int tn, const RowNode& rn) {
      const std::string n = std::to_string(EPL);
      max_bytes = std::max(max_bytes, dealt ? 4 * prec_bytes(rn.prec) : std::min(16, EPL * prec_bytes(rn.prec)));
      const std::string lane = dealt ? "b200_t, " : "";
      if (rn.prec == Prec::Single) return std::string("    b200_ld_row") + (dealt ? "v<" : "<") + n + ">(" + row_ptr(tn, rn) + ", " + lane + reg(tn) + ");\n";
      return std::string("    b200_ld_row") + (dealt ? "v16<" : "16<") + n + ", " + (rn.prec == Prec::Half ? "true" : "false") + ">(" + row_ptr(tn, rn) + ", " + lane + reg(tn) + ");\n";
    };
    auto stv = [&](int tn, const RowNode& rn) {
      const std::string n = std::to_string(EPL);
      max_bytes = std::max(max_bytes, dealt ? 4 * prec_bytes(rn.prec) : std::min(16, EPL * prec_bytes(rn.prec)));
      const std::string lane = dealt ? "b200_t, " : "";
      if (rn.prec == Prec::Single) return std::string("    b200_st_row") + (dealt ? "v<" : "<") + n + ">(" + row_ptr(tn, rn) + ", " + lane + reg(tn) + ");\n";
      return std::string("    b200_st_row") + (dealt ? "v16<" : "16<") + n + ", " + (rn.prec == Prec::Half ? "true" : "false") + ">(" + row_ptr(tn, rn) + ", " + lane + reg(tn) + ");\n";
    };
    // rows that are the same for every row of the kernel (a scale, a shift: no row symbol in their
    // position) are loaded once per warp, before the loop over the warp's rows
    auto row_invariant = [&](const RowNode& rn) {
      if (rn.produced) return false;
      for (auto& ix : rn.idcs)
        if (ix.kind != Index::Fixed) return false;
      return true;
    };
    std::string text, decls, pre_decls, pre_text;
    bool any_invariant = false;
    for (auto& kv : rownodes) {
      const std::string d = "    float " + reg(kv.first) + "[" + std::to_string(EPL) + "];\n";
      if (row_invariant(kv.second)) { pre_decls += d; any_invariant = true; }
      else decls += d;
    }
    std::set<int> have;
    auto forwards = [&]() {
      em.row_forwards.clear();
      for (auto& kv : rownodes) {
        Indices idcs = kv.second.idcs;
        Index any;
        idcs.push_back(any);
        em.row_forwards.push_back({kv.first, idcs, (int)idcs.size() - 1, reg(kv.first), " - b200_t0", "b200_e"});   // (every element loop below runs over b200_e)
      }
    };
    forwards();
    for (size_t k = 0; k < stages.size(); ++k) {
      const RegRowStage& st = stages[k];
      const Stmt& set = *st.set;
      const Tnode& T = code.prog.tn(set.tn);
      // rows this stage reads that are not in registers yet
      walk_scalar(*set.value, [&](const Scalar& e) {
        if (e.kind != Scalar::Get) return;
        auto it = rownodes.find(e.tn);
        if (it == rownodes.end() || it->second.produced || have.count(e.tn)) return;
        bool positional = !e.idcs.empty() && e.idcs.back().kind == Index::Iter &&
                          (e.idcs.back().sym == st.t_sym || std::count(st.scope_syms.begin(), st.scope_syms.end(), e.idcs.back().sym));
        if (!positional) return;
        if (row_invariant(it->second)) pre_text += ld(e.tn, it->second);
        else text += ld(e.tn, it->second);
        have.insert(e.tn);
      }, [](const Stmt&) {});
      if (st.coop) {
        text += "    {\n";
        size_t si = 0;
        std::function<void(const Scalar&)> rec = [&](const Scalar& e) {
          if (e.kind == Scalar::LocalScope) {
            std::string op;
            for (auto& sc : st.scopes)
              if (sc.first == e.scope_id) op = sc.second;
            const Prec p = code.prog.tn(e.tn).prec;
            const Stmt* b = e.body.get();
            if (b->kind == Stmt::Seq) b = b->items[1].get();
            const std::string name = em.scope_name(e.scope_id, e.tn);
            const double neutral = op == "add" ? 0.0 : (op == "max" ? -INFINITY : INFINITY);
            text += "      " + std::string(Emitter::ctype(p)) + " " + name + " = " + em.constant(neutral, p) + ";\n";
            text += "#pragma unroll\n      for (unsigned int b200_e = 0; b200_e < " + std::to_string(EPL) + "u; ++b200_e) {\n"
                    "        const unsigned int " + b->index + " = " + own + ";\n" + em.stmt(*b->body, 8) + "      }\n";
            text += "      " + name + " = b200_warp_" + (op == "add" ? std::string("sum") : op) + "(" + name + ");\n";
            em.scope_subst[e.scope_id] = name;
            ++si;
            return;
          }
          for (auto& a : e.args) rec(*a.s);
        };
        rec(*set.value);
        Emitter::Res v = em.scalar(T.prec, *set.value);
        em.scope_subst.clear();
        const std::string sname = "b200_val" + std::to_string(set.tn);
        decls += "    " + std::string(Emitter::rtype(T.prec)) + " " + sname + ";\n";
        text += "      " + sname + " = " + v.expr + ";\n";
        text += "      if (b200_t == 0u) " + T.ident + "[" + em.offset(set.idcs, T.dims) + "] = " + Emitter::store_wrap(T.prec, sname) + ";\n";
        text += "    }\n";
        em.forwarded[set.tn] = {set.idcs, sname};     // every lane holds the value after the shuffle tree
      } else {
        em.set_redirect[set.tn] = {set.idcs, reg(set.tn) + "[b200_e]"};
        const std::string loop_head = "#pragma unroll\n    for (unsigned int b200_e = 0; b200_e < " + std::to_string(EPL) + "u; ++b200_e) {\n"
                                      "      const unsigned int " + st.t_sym + " = " + own + ";\n";
        // divisors that are the same for the whole row (a standard deviation, a sum) are prepared
        // once: reciprocal and range check per row, a short exact sequence per element
        std::vector<std::string> probe;
        em.divisor_probe = &probe;
        const std::string body_plain = em.stmt(set, 6);
        em.divisor_probe = nullptr;
        std::vector<std::string> inv;
        for (auto& d : probe)
          if (d.find('[') == std::string::npos && d.find(st.t_sym) == std::string::npos && d.find("b200_e") == std::string::npos &&
              std::find(inv.begin(), inv.end(), d) == inv.end())
            inv.push_back(d);
        if (!inv.empty()) {
          std::string all_fast;
          text += "    {\n";
          for (size_t q = 0; q < inv.size(); ++q) {
            const std::string nm = "b200_dv" + std::to_string(set.tn) + "_" + std::to_string(q);
            text += "    const b200_divisor " + nm + " = b200_divisor_of(" + inv[q] + ");\n";
            em.divisor_vars[inv[q]] = nm;
            all_fast += (q ? " && " : "") + nm + ".fast";
          }
          const std::string body_fast = em.stmt(set, 6);
          em.divisor_vars.clear();
          text += "    if (" + all_fast + ") {\n" + loop_head + body_fast + "    }\n    } else {\n" + loop_head + body_plain + "    }\n    }\n    }\n";
        } else {
          text += loop_head + body_plain + "    }\n";
        }
        em.set_redirect.erase(set.tn);
        text += stv(set.tn, rownodes[set.tn]);
        have.insert(set.tn);
      }
    }
    f.min_align = max_bytes;
    std::string statics = static_prologue(text, em, 2);
    std::ostringstream k_src;
    k_src << "extern \"C\" __global__ void __launch_bounds__(" << f.block << ") " << f.kernel << "(";
    emit_params(k_src, f, em, written);
    k_src << ") {\n" << kGridEntry << statics
          << "  const unsigned int b200_t = threadIdx.x & 31u;\n  const unsigned int b200_t0 = b200_t * " << EPL << "u;\n"
          << "  const unsigned long long b200_warp = ((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;\n"
          << "  const unsigned long long b200_nwarps = ((unsigned long long)gridDim.x * blockDim.x) >> 5;\n"
          << pre_decls << pre_text
          << "  for (unsigned long long b200_row = b200_warp; b200_row < " << rows << "ull; b200_row += b200_nwarps) {\n";
    {
      std::string rem = "b200_row";
      for (size_t q = L; q-- > 0;) {
        const std::string ext = std::to_string(first.par[q].extent()) + "ull";
        k_src << "    const unsigned int " << canon[q] << " = (unsigned int)" << (q == 0 ? rem : "(" + rem + " % " + ext + ")") << ";\n";
        if (q != 0) {
          k_src << "    const unsigned long long b200_q" << q << " = " << rem << " / " << ext << ";\n";
          rem = "b200_q" + std::to_string(q);
        }
      }
    }
    k_src << decls << text << "  }\n}\n\n";
    src << k_src.str();
    // with rows loaded once per warp, a warp takes several rows: as many blocks as stay resident on 148
    // SMs (three of 256 threads at this kernel's register use), each warp striding over the rows
    if (any_invariant && rows >= 2 * 148 * 3 * 8) f.grid_override = 148 * 3;
    f.note = "row-fused " + std::to_string(run.size()) + " stages, one warp per row, rows in registers (" + std::to_string(EPL) +
             " elements per lane" + (dealt ? ", dealt four at a time" : "") + ")";
    *out = f;
    return true;
  }

  // Row fusion.  Consecutive stages whose outermost parallel loop has the same extent, and which
  // hand data to one another only within one iteration of that loop (every node written by one
  // of them and touched by another is indexed by the row symbol on one fixed axis, nowhere else),
  // run as ONE kernel: a thread takes a row and executes the stages one after the other for it,
  // the inner parallel loops of each stage becoming short serial loops.  A softmax over ten
  // logits (row max, exponentials, row sum) is one launch and one pass instead of three.
  bool rows_independent(const std::vector<size_t>& run) {
    std::map<int, int> writers, users;  // node -> number of stages writing / touching it
    for (size_t i : run) {
      const Piece& pc = pieces[i];
      for (int n : pc.written) writers[n]++;
      for (int n : pc.used) users[n]++;
    }
    std::map<int, int> axis;  // shared node -> axis that carries the row symbol
    bool ok = true;
    for (size_t i : run) {
      const Piece& pc = pieces[i];
      auto check = [&](int tn, const Indices& idcs) {
        if (!writers.count(tn) || users[tn] < 2) return;   // private to one stage, or only read
        int a = -1;
        for (size_t k = 0; k < idcs.size(); ++k) {
          if (idcs[k].kind == Index::Iter && idcs[k].sym == pc.row_sym && a < 0) a = (int)k;
          else if (idcs[k].uses(pc.row_sym)) ok = false;
        }
        if (a < 0) { ok = false; return; }
        auto it = axis.find(tn);
        if (it == axis.end()) axis[tn] = a;
        else if (it->second != a) ok = false;
      };
      walk_stmt(
          *pc.body,
          [&](const Scalar& e) {
            if (e.kind == Scalar::Get) check(e.tn, e.idcs);
            if (e.kind == Scalar::GetDyn && writers.count(e.tn) && users[e.tn] >= 2) ok = false;
          },
          [&](const Stmt& st) {
            if (st.kind == Stmt::Set) {
              if (st.vec_len > 0 && writers.count(st.tn) && users[st.tn] >= 2) ok = false;
              check(st.tn, st.idcs);
            }
            if (st.kind == Stmt::ZeroOut) ok = false;
          });
    }
    return ok;
  }

  Stage emit_rows(const std::vector<size_t>& run) {
    Stage f;
    merge_origins(f, run);
    f.kind = Stage::Generic;
    f.kernel = code.stages[run.front()].kernel;
    f.block = 128;
    f.total = pieces[run.front()].rows;
    Emitter em(code.prog);
    std::set<int> written;
    std::string text;
    for (size_t i : run) {
      const Stage& st = code.stages[i];
      const Piece& pc = pieces[i];
      f.min_align = std::max(f.min_align, st.min_align);
      em.used_nodes.insert(pc.used.begin(), pc.used.end());
      written.insert(pc.written.begin(), pc.written.end());
      em.uses_merge |= pc.uses_merge;
      const std::string inner = std::to_string(st.total / pc.rows) + "ull";
      text += "    for (unsigned long long b200_g = b200_row * " + inner + "; b200_g < (b200_row + 1ull) * " + inner +
              "; ++b200_g) {\n" + pc.decomp + pc.body_text + "    }\n";
    }
    std::string statics = static_prologue(text, em, 2);
    std::ostringstream k_src;
    k_src << "extern \"C\" __global__ void __launch_bounds__(" << f.block << ") " << f.kernel << "(";
    emit_params(k_src, f, em, written);
    k_src << ") {\n" << kGridEntry << statics
          << "  for (unsigned long long b200_row = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; b200_row < "
          << f.total << "ull; b200_row += (unsigned long long)gridDim.x * blockDim.x) {\n"
          << text << "  }\n}\n\n";
    src << k_src.str();
    f.note = "row-fused " + std::to_string(run.size()) + " stages, one thread per row";
    return f;
  }

  // Pointwise chain.  Consecutive stages over the SAME parallel loops (no serial loops, no
  // cooperative reductions) that hand data to one another only at one position of those loops
  // run as one kernel: a thread executes the stages one after the other for its element (or
  // pair).  What one stage stores the next reads back from L1 / L2 instead of DRAM, and a
  // momentum SGD step (delta, momentum, Nesterov correction, parameter) is one launch per
  // parameter instead of four.
  bool pointwise_member(size_t i, const Piece* like) {
    auto it = pieces.find(i);
    if (it == pieces.end() || !it->second.any_body) return false;
    const Piece& pc = it->second;
    if (pc.coop != 0 || pc.ser_work != 1 || pc.par.empty() || code.stages[i].total <= 0) return false;
    for (auto& d : pc.par)
      if (d.from != 0) return false;
    if (like) {
      if (pc.par.size() != like->par.size() || pc.pairs != like->pairs) return false;
      for (size_t q = 0; q < pc.par.size(); ++q)
        if (pc.par[q].extent() != like->par[q].extent()) return false;
    }
    return true;
  }

  Stage emit_pointwise_chain(const std::vector<size_t>& run) {
    Stage f = code.stages[run.front()];
    merge_origins(f, run);
    Emitter em(code.prog);
    std::set<int> written;
    std::string text;
    for (size_t i : run) {
      const Piece& pc = pieces[i];
      f.min_align = std::max(f.min_align, code.stages[i].min_align);
      em.used_nodes.insert(pc.used.begin(), pc.used.end());
      written.insert(pc.written.begin(), pc.written.end());
      em.uses_merge |= pc.uses_merge;
      text += "    {\n" + pc.decomp + pc.body_text + "    }\n";
    }
    std::string statics = static_prologue(text, em, 2);
    std::ostringstream k_src;
    k_src << "extern \"C\" __global__ void __launch_bounds__(" << f.block << ") " << f.kernel << "(";
    emit_params(k_src, f, em, written);
    k_src << ") {\n" << kGridEntry << statics
          << "  for (unsigned long long b200_g = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; b200_g < "
          << f.total << "ull; b200_g += (unsigned long long)gridDim.x * blockDim.x) {\n"
          << text << "  }\n}\n\n";
    src << k_src.str();
    f.note = "pointwise chain of " + std::to_string(run.size()) + " stages" + (pieces[run.front()].pairs ? ", pairs" : "");
    return f;
  }

  // Decides which stages share a launch and writes the kernels' text.
  void emit_kernels() {
    {
      // zero_outs that later stages made unnecessary leave the list (pieces are keyed by stage index)
      std::vector<Stage> kept;
      std::map<size_t, Piece> moved;
      for (size_t i = 0; i < code.stages.size(); ++i) {
        if (code.stages[i].kind == Stage::Memset && code.stages[i].memset_tn < 0) continue;
        auto it = pieces.find(i);
        if (it != pieces.end()) moved[kept.size()] = it->second;
        kept.push_back(code.stages[i]);
      }
      code.stages.swap(kept);
      pieces.swap(moved);
    }
    std::vector<Stage> out;
    auto fusable = [&](size_t i) {
      const Stage& st = code.stages[i];
      if (st.kind == Stage::Memset) {
        const Tnode& t = code.prog.tn(st.memset_tn);
        return opt.enable_fuse && t.bytes() <= 262144 && prec_bytes(t.prec) <= 8 && t.prec != Prec::Uint4x32;
      }
      auto it = pieces.find(i);
      return it != pieces.end() && it->second.fusable;
    };
    auto row_candidate = [&](size_t i) {
      auto it = pieces.find(i);
      return it != pieces.end() && it->second.body && it->second.rows >= 256 && it->second.per_row <= 64;
    };
    for (size_t i = 0; i < code.stages.size();) {
      if (opt.enable_fuse && pieces.count(i) && pieces[i].any_body && (pieces[i].coop == 0 || pieces[i].coop == 32)) {
        // the row is given by the first warp-cooperative stage of the run
        size_t L = 0;
        for (size_t j = i; j < code.stages.size() && j < i + 16; ++j) {
          auto it = pieces.find(j);
          if (it == pieces.end()) break;
          if (it->second.coop == 32) { L = it->second.par.size(); break; }
          if (it->second.coop != 0) break;
        }
        if (L > 0 && warp_row_member(i, L, nullptr)) {
          const Piece& first = pieces[i];
          int64_t rows = 1;
          for (size_t q = 0; q < L; ++q) rows *= first.par[q].extent();
          std::vector<size_t> run = {i};
          bool has_coop = first.coop == 32;
          size_t j = i + 1;
          while (j < code.stages.size() && run.size() < 16 && warp_row_member(j, L, &first)) {
            run.push_back(j);
            if (!rows_independent_prefix(run, L)) { run.pop_back(); break; }
            has_coop = has_coop || pieces[j].coop == 32;
            ++j;
          }
          // a trailing pointwise stage gains nothing from the warp form unless it follows a reduction
          if (run.size() >= 2 && has_coop && rows >= 128) {
            Stage reg_form;
            if (emit_warp_rows_reg(run, L, &reg_form)) out.push_back(reg_form);
            else out.push_back(emit_warp_rows(run, L));
            i = run.back() + 1;
            continue;
          }
        }
      }
      if (row_candidate(i)) {
        // the longest run that stays row-independent; runs made only of small stages are left to
        // the single-block fusion below, which also takes stages of unrelated shapes
        std::vector<size_t> run = {i};
        size_t j = i + 1;
        bool all_small = fusable(i);
        while (j < code.stages.size() && row_candidate(j) && pieces[j].rows == pieces[i].rows && run.size() < 16) {
          run.push_back(j);
          if (!rows_independent(run)) { run.pop_back(); break; }
          all_small = all_small && fusable(j);
          ++j;
        }
        if (run.size() >= 2 && !all_small) {
          out.push_back(emit_rows(run));
          i = run.back() + 1;
          continue;
        }
      }
      if (opt.enable_fuse && !fusable(i) && pointwise_member(i, nullptr)) {
        const Piece& first = pieces[i];
        std::vector<size_t> run = {i};
        size_t j = i + 1;
        while (j < code.stages.size() && run.size() < 8 && pointwise_member(j, &first)) {
          run.push_back(j);
          if (!rows_independent_prefix(run, first.par.size())) { run.pop_back(); break; }
          ++j;
        }
        if (run.size() >= 2) {
          out.push_back(emit_pointwise_chain(run));
          i = run.back() + 1;
          continue;
        }
      }
      if (fusable(i)) {
        std::vector<size_t> run;
        size_t j = i;
        while (j < code.stages.size() && fusable(j)) run.push_back(j++);
        int kernels = 0;
        for (size_t k : run) kernels += code.stages[k].kind != Stage::Memset;
        if (run.size() >= 2 && kernels >= 1) {
          out.push_back(emit_fused(run));
          i = j;
          continue;
        }
      }
      Stage st = code.stages[i];
      auto it = pieces.find(i);
      if (it != pieces.end()) emit_single(st, it->second);
      out.push_back(st);
      ++i;
    }
    code.stages = out;
  }

  // A group of threads per output element: each Local_scope reduction runs over its flattened
  // loop space strided by the group width, partial results are combined with shuffles (and
  // shared memory across warps), and thread 0 of the group evaluates and stores the rest.
  std::string coop_body(Emitter& em, const Stmt& set, const CoopInfo& ci, int ind) {
    std::string out;
    std::string padding((size_t)ind, ' ');
    const Tnode& t = code.prog.tn(set.tn);
    std::function<void(const Scalar&)> rec = [&](const Scalar& e) {
      if (e.kind == Scalar::LocalScope) {
        std::string op;
        for (auto& s : ci.scopes)
          if (s.first == e.scope_id) op = s.second;
        Prec p = code.prog.tn(e.tn).prec;
        const Stmt& b = *e.body;
        const Stmt* loop = b.kind == Stmt::For ? &b : b.items[1].get();
        std::vector<LoopDim> red;
        const Stmt* inner = loop;
        while (inner->kind == Stmt::For) {
          red.push_back({inner->index, inner->from, inner->to});
          inner = inner->body.get();
        }
        int64_t total = 1;
        for (auto& d : red) total *= d.extent();
        std::string name = em.scope_name(e.scope_id, e.tn);
        double neutral = op == "add" ? 0.0 : (op == "max" ? -INFINITY : INFINITY);
        out += padding + Emitter::ctype(p) + " " + name + " = " + em.constant(neutral, p) + ";\n";
        std::string lv = "b200_l" + std::to_string(e.scope_id);
        const bool narrow = total < (1ll << 31);
        const std::string IT = narrow ? "unsigned int" : "unsigned long long", SUF = narrow ? "u" : "ull";
        out += padding + "for (" + IT + " " + lv + " = b200_t; " + lv + " < " + std::to_string(total) + SUF + "; " + lv +
               " += " + std::to_string(ci.width) + "u) {\n";
        std::string rem = lv;
        for (size_t i = red.size(); i-- > 0;) {
          const LoopDim& d = red[i];
          std::string ext = std::to_string(d.extent()) + SUF;
          std::string val = i == 0 ? rem : "(" + rem + " % " + ext + ")";
          out += padding + "  const unsigned int " + d.sym + " = (unsigned int)" + val +
                 (d.from ? " + " + std::to_string(d.from) : std::string()) + ";\n";
          if (i != 0) {
            std::string nr = "b200_q" + std::to_string(e.scope_id) + "_" + std::to_string(i);
            out += padding + "  const " + IT + " " + nr + " = " + rem + " / " + ext + ";\n";
            rem = nr;
          }
        }
        out += em.stmt(*inner, ind + 2);
        out += padding + "}\n";
        const std::string fn = op == "add" ? "sum" : op;
        if (ci.width > 32) out += padding + name + " = b200_block_" + fn + "(" + name + ", b200_red);\n";
        else out += padding + name + " = b200_warp_" + fn + "(" + name + ");\n";
        em.scope_subst[e.scope_id] = name;
        return;
      }
      for (auto& a : e.args) rec(*a.s);
    };
    rec(*set.value);
    Emitter::Res v = em.scalar(t.prec, *set.value);
    em.used_nodes.insert(set.tn);
    out += padding + "if (b200_t == 0) " + t.ident + "[" + em.offset(set.idcs, t.dims) + "] = " + Emitter::store_wrap(t.prec, v.expr) + ";\n";
    em.scope_subst.clear();
    return out;
  }

  // A node that a later stage only tests against zero (the mask of an attention stage), packed to
  // one bit per element in element order: bit (i % 32) of word (i / 32) = (node[i] != 0).  The bits
  // live in the routine's scratch; for a read-only node they are made once per run and shared by
  // every stage that asks for them.  Returns the byte offset in the reduction scratch.
  std::map<int, size_t> packed_bits;
  size_t pack_bits_stage(int tn) {
    const Tnode& t = code.prog.tn(tn);
    if (t.read_only) {
      auto it = packed_bits.find(tn);
      if (it != packed_bits.end()) return it->second;
    }
    const long long words = (t.num_elems() + 31) / 32;
    const size_t off = code.reduce_scratch_bytes;
    code.reduce_scratch_bytes = (code.reduce_scratch_bytes + (size_t)words * 4 + 255) & ~(size_t)255;
    Stage st;
    st.kind = Stage::Generic;
    st.kernel = kernel_name();
    st.args = {{KArg::Node, tn}, {KArg::Scratch, (int)off}};
    st.total = words * 32;
    st.block = 256;
    st.note = "one bit per element: (value != 0), for the stages that only test this node";
    src << "extern \"C\" __global__ void __launch_bounds__(256) " << st.kernel << "(const " << Emitter::ctype(t.prec) << "* __restrict__ "
        << t.ident << ", unsigned char* b200_bits) {\n" << kGridEntry
        << "  unsigned int* b200_words = (unsigned int*)b200_bits;\n"
        << "  for (unsigned long long b200_i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; b200_i < " << words * 32
        << "ull; b200_i += (unsigned long long)gridDim.x * blockDim.x) {\n"
        << "    const bool b200_nz = b200_i < " << t.num_elems() << "ull && " << Emitter::load_wrap(t.prec, t.ident + "[b200_i]") << " != 0;\n"
        << "    const unsigned int b200_w = __ballot_sync(0xffffffffu, b200_nz);\n"
        << "    if ((threadIdx.x & 31u) == 0u) b200_words[b200_i >> 5] = b200_w;\n  }\n}\n\n";
    code.stages.push_back(st);
    if (t.read_only) packed_bits[tn] = off;
    return off;
  }

  // an epilogue that ends in a grid-wide sum keeps its per-warp partials and its ticket in the
  // routine's reduction scratch (zeroed at link; the kernel resets its ticket itself)
  void assign_epilogue_scratch(Stage& g) {
    if (!g.epi_scratch_bytes) return;
    for (auto& a : g.args)
      if (a.kind == KArg::Scratch) a.tn = (int)code.reduce_scratch_bytes;
    code.reduce_scratch_bytes += g.epi_scratch_bytes;
    code.reduce_scratch_bytes = (code.reduce_scratch_bytes + 255) & ~(size_t)255;
  }

  // Range-checked build.  Every generic kernel's node pointers are renamed and shadowed by a
  // b200_checked proxy of the node's size (kernels/numerics.cuh), so that each `node[offset]` the
  // emitters wrote is compared with the number of elements the node has; the kernels get the device
  // status word as a last parameter.
  void apply_bounds() {
    std::string text = code.source;
    for (auto& st : code.stages) {
      if (st.kind != Stage::Generic || st.kernel.empty()) continue;
      const std::string head = " " + st.kernel + "(";
      size_t h = text.find(head);
      if (h == std::string::npos) continue;
      const size_t p0 = h + head.size();
      const size_t p1 = text.find(") {\n", p0);
      if (p1 == std::string::npos) continue;
      std::string params = text.substr(p0, p1 - p0), proxies;
      for (auto& t : code.prog.tnodes) {
        if (t.mode == Mode::Virtual) continue;
        // "<type>* [__restrict__ ]ident" followed by ',' or the end
        for (const std::string& sep : {std::string("* __restrict__ "), std::string("* ")}) {
          const std::string needle = sep + t.ident;
          size_t q = 0;
          while ((q = params.find(needle, q)) != std::string::npos) {
            const size_t end = q + needle.size();
            if (end != params.size() && params[end] != ',') { q = end; continue; }
            size_t b = params.rfind(',', q);
            b = b == std::string::npos ? 0 : b + 1;
            while (b < q && params[b] == ' ') ++b;
            const std::string type = params.substr(b, q - b);
            params.insert(end, "__p");
            proxies += "  const b200_checked<" + type + "> " + t.ident + " = {" + t.ident + "__p, " + std::to_string(t.num_elems()) +
                       "ull, b200_status, " + std::to_string(t.id) + "u};\n";
            q = end + 3;
          }
        }
      }
      params += (params.empty() ? "" : ", ") + std::string("unsigned int* b200_status");
      text.replace(p0, p1 - p0, params);
      const size_t body = text.find(") {\n", p0) + 4;
      text.insert(body, proxies);
      st.args.push_back({KArg::Status, -1});
    }
    code.source = text;
  }

  void memset_stage(int tn) {
    Stage st;
    st.kind = Stage::Memset;
    st.memset_tn = tn;
    st.note = "zero_out";
    st.writes = {tn};
    code.stages.push_back(st);
  }

  void top_level(const StmtP& s, std::vector<StmtP>& flat) {
    if (s->kind == Stmt::Seq)
      for (auto& x : s->items) top_level(x, flat);
    else if (s->kind != Stmt::Noop && s->kind != Stmt::Comment)
      flat.push_back(s);
  }

  // the perfect-nest pointwise assignments that directly follow position `from`
  std::vector<Follower> followers_after(const std::vector<StmtP>& flat, size_t from) {
    std::vector<Follower> out;
    for (size_t k = from; k < flat.size() && out.size() < 8; ++k) {
      Follower f;
      const Stmt* b = flat[k].get();
      while (b->kind == Stmt::For) {
        f.nest.push_back({b->index, b->from, b->to});
        b = b->body.get();
      }
      if (b->kind != Stmt::Set) break;
      f.set = b;
      out.push_back(f);
    }
    return out;
  }

  // Function-scope scalar locals.  `hoist_cross_statement_cse` (arrayjit/lib/low_level.ml:2039-2135)
  // turns a Local_scope shared by sibling assignments into `Declare_local id; <the scope's body>`
  // before the first user, the users reading `Get_local id`; the cc backend prints a function-scope
  // variable (arrayjit/lib/c_syntax.ml:695-704,730-734).  Siblings inside one loop body stay inside
  // one kernel and need nothing.  At the top level of the routine the users become different
  // kernels, so the local becomes a one-element routine-local node: declaration and body turn back
  // into `t[0] := scope { body }` (which the reduction paths recognise) and every later
  // `Get_local id` into `t[0]`.  The value makes one round trip through memory in its own precision.
  void unhoist_function_locals(std::vector<StmtP>& flat) {
    std::map<int, int> hoisted;   // scope id -> synthetic node id
    auto writes_scope = [](const Stmt& s, int sid) {
      bool w = false;
      walk_stmt(s, [](const Scalar&) {}, [&](const Stmt& x) { if (x.kind == Stmt::SetLocal && x.scope_id == sid) w = true; });
      return w;
    };
    int next_id = 0;
    for (auto& t : code.prog.tnodes) next_id = std::max(next_id, t.id + 1);
    std::vector<StmtP> out;
    for (size_t i = 0; i < flat.size(); ++i) {
      const StmtP& s = flat[i];
      if (s->kind != Stmt::DeclareLocal) { out.push_back(s); continue; }
      const Tnode& st = code.prog.tn(s->tn);
      Tnode syn;
      syn.id = next_id++;
      syn.ident = "b200_local" + std::to_string(s->scope_id) + "_" + st.ident;
      syn.prec = st.prec;
      syn.dims = {1};
      syn.mode = Mode::Local;
      syn.zero_init = s->needs_init;
      auto body = std::make_shared<Stmt>();
      body->kind = Stmt::Seq;
      size_t j = i + 1;
      while (j < flat.size() && writes_scope(*flat[j], s->scope_id)) body->items.push_back(flat[j++]);
      hoisted[s->scope_id] = syn.id;
      code.prog.tn_index[syn.id] = code.prog.tnodes.size();
      code.prog.tnodes.push_back(syn);
      if (!body->items.empty()) {
        auto scope = std::make_shared<Scalar>();
        scope->kind = Scalar::LocalScope;
        scope->scope_id = s->scope_id;
        scope->tn = s->tn;
        scope->body = body;
        auto set = std::make_shared<Stmt>();
        set->kind = Stmt::Set;
        set->tn = syn.id;
        Index zero;
        set->idcs = {zero};
        set->value = scope;
        out.push_back(set);
      }
      i = j - 1;
    }
    if (hoisted.empty()) return;
    // every remaining mention of a hoisted scope reads the node
    std::function<ScalarP(const ScalarP&, int)> fix_scalar;
    std::function<StmtP(const StmtP&, int)> fix_stmt = [&](const StmtP& s, int inside) -> StmtP {
      auto c = std::make_shared<Stmt>(*s);
      for (auto& x : c->items) x = fix_stmt(x, inside);
      if (c->body) c->body = fix_stmt(c->body, inside);
      if (c->value) c->value = fix_scalar(c->value, inside);
      if (c->kind == Stmt::SetLocal && c->scope_id != inside && hoisted.count(c->scope_id))
        throw Error(-4, "a function-scope local is assigned after its defining statements");
      return c;
    };
    fix_scalar = [&](const ScalarP& e, int inside) -> ScalarP {
      if (e->kind == Scalar::GetLocal && e->scope_id != inside && hoisted.count(e->scope_id)) {
        auto g = std::make_shared<Scalar>();
        g->kind = Scalar::Get;
        g->tn = hoisted[e->scope_id];
        Index zero;
        g->idcs = {zero};
        return g;
      }
      auto c = std::make_shared<Scalar>(*e);
      // inside the re-wrapped body the scope's own id keeps meaning the local variable
      const int in = (c->kind == Scalar::LocalScope && hoisted.count(c->scope_id)) ? c->scope_id : inside;
      if (c->body) c->body = fix_stmt(c->body, in);
      for (auto& a : c->args) a.s = fix_scalar(a.s, in);
      return c;
    };
    for (auto& s : out) s = fix_stmt(s, -1);
    flat.swap(out);
  }

  void run() {
    std::vector<StmtP> flat;
    top_level(code.prog.body, flat);
    unhoist_function_locals(flat);
    src << kNumericsSource << "\n";
    std::set<int> zeroed;  // nodes zeroed by the previous stage (for beta = 0 contractions)
    std::map<int, size_t> zero_stage;  // ... and the index of the stage that zeroes them
    std::set<int> zero_read;           // zeroed nodes some later stage has read as zeros
    auto drop_zero_out = [&](int tn) {
      // the node is about to be overwritten completely by a stage that does not read it
      auto it = zero_stage.find(tn);
      if (it == zero_stage.end() || zero_read.count(tn)) return;
      code.stages[it->second].memset_tn = -1;   // filtered out in emit_kernels
      zero_stage.erase(it);
    };
    // plans the statement at flat[i]; advances i past the statements it absorbed
    auto plan_one = [&](size_t& i) {
      const StmtP& s = flat[i];
      if (s->kind == Stmt::DeclareLocal || s->kind == Stmt::SetLocal)
        throw Error(-4, "a function-scope scalar local is assigned away from its declaration");
      if (s->kind == Stmt::ZeroOut) {
        const Tnode& t = code.prog.tn(s->tn);
        if (t.mode == Mode::Virtual) return;
        // a zero_out that a following contraction absorbs (beta = 0) is dropped below
        bool absorbed = false;
        if (gemm_at(i + 1) && i + 1 < flat.size() && flat[i + 1]->kind == Stmt::For) {
          std::vector<LoopDim> nest;
          StmtP body = flat[i + 1];
          while (body->kind == Stmt::For) {
            nest.push_back({body->index, body->from, body->to});
            body = body->body;
          }
          Stage g;
          int n_fused = 0;
          if (body->kind == Stmt::Set && body->tn == s->tn &&
              match_gemm(code.prog, nest, *body, true, opt, followers_after(flat, i + 2), &n_fused, &g)) {
            if (g.gemm.split_k > 1) memset_stage(s->tn);   // partial tiles are added to the zeroed node
            assign_epilogue_scratch(g);
            g.kernel = kernel_name();
            g.gemm_source = gemm_translation_unit(code.prog, g, g.kernel, opt);
            code.stages.push_back(g);
            absorbed = true;
            i += 1 + (size_t)n_fused;
          }
        }
        if (!absorbed) {
          zero_stage[s->tn] = code.stages.size();
          zero_read.erase(s->tn);
          memset_stage(s->tn);
          zeroed.insert(s->tn);  // still all zero until some stage writes it
        }
        return;
      }
      // peel the perfect loop nest
      std::vector<LoopDim> nest;
      StmtP body = s;
      while (body->kind == Stmt::For) {
        nest.push_back({body->index, body->from, body->to});
        body = body->body;
      }
      if (!body_has_set(*body)) return;
      {
        std::set<std::pair<int, int>> declared, used;
        collect_scopes(*body, declared, used);
        for (auto& u : used)
          if (!declared.count(u))
            throw Error(-4, "a scalar local is read outside the statement that defines it");
      }
      // a node zeroed earlier and untouched since lets a contraction skip reading it (beta = 0)
      std::set<int> writes_now;
      walk_stmt(*body, [](const Scalar&) {}, [&](const Stmt& w) {
        if (w.kind == Stmt::Set || w.kind == Stmt::ZeroOut) writes_now.insert(w.tn);
      });
      const bool was_zero = body->kind == Stmt::Set && zeroed.count(body->tn) > 0;
      walk_stmt(*body, [&](const Scalar& e) {
        if ((e.kind == Scalar::Get || e.kind == Scalar::GetDyn) && zeroed.count(e.tn) && !(body->kind == Stmt::Set && e.tn == body->tn))
          zero_read.insert(e.tn);
      }, [](const Stmt&) {});
      for (int w : writes_now) zeroed.erase(w);
      if (opt.enable_attn && gemm_at(i) && body->kind == Stmt::Set && i + 6 <= flat.size()) {
        // scores, softmax and weights . values as one kernel
        bool allowed = true;
        for (size_t k = i; k < i + 6; ++k) allowed = allowed && gemm_at(k);
        Stage a;
        int n_abs = 0;
        if (allowed && match_attention(code.prog, flat, i, opt, &n_abs, &a)) {
          for (int w : a.writes) zeroed.erase(w);
          // masks as bits: one packing stage per mask node (shared when the node is read-only)
          {
            size_t k = 0;
            for (auto& arg : a.args)
              if (arg.kind == KArg::Scratch) arg.tn = (int)pack_bits_stage(a.attn.cond_tns.at(k++));
          }
          a.kernel = kernel_name();
          a.gemm_source = attn_translation_unit(code.prog, a, a.kernel);
          code.stages.push_back(a);
          i += (size_t)n_abs - 1;
          return;
        }
      }
      if (gemm_at(i) && body->kind == Stmt::Set) {
        Stage g;
        int n_fused = 0;
        const std::vector<Follower> fol = followers_after(flat, i + 1);
        if (match_gemm(code.prog, nest, *body, was_zero, opt, fol, &n_fused, &g)) {
          for (int f = 0; f < n_fused; ++f) zeroed.erase(fol[(size_t)f].set->tn);
          // beta = 0 over the whole node: the zero_out before it has no reader left
          if (was_zero && !g.gemm.accumulate && g.gemm.split_k == 1 && covers_node(*body, nest)) drop_zero_out(body->tn);
          assign_epilogue_scratch(g);
          g.kernel = kernel_name();
          g.gemm_source = gemm_translation_unit(code.prog, g, g.kernel, opt);
          code.stages.push_back(g);
          i += (size_t)n_fused;
          return;
        }
      }
      if (generic_stage(nest, body, was_zero)) drop_zero_out(body->tn);
    };
    for (size_t i = 0; i < flat.size(); ++i) {
      const size_t before = code.stages.size(), first = i;
      cur_origin = (int)i;
      plan_one(i);
      for (size_t k = before; k < code.stages.size(); ++k)
        for (size_t o = first; o <= i; ++o) code.stages[k].origins.push_back((int)o);
    }
    emit_kernels();
    code.source = src.str();
    if (opt.bounds) apply_bounds();
    // routine-local nodes that some stage touches get scratch (a node whose every use was fused
    // away, such as the score matrix of a fused attention stage, needs none)
    std::set<int> touched;
    for (auto& st : code.stages) {
      if (st.kind == Stage::Memset) touched.insert(st.memset_tn);
      for (auto& a : st.args)
        if (a.kind == KArg::Node) touched.insert(a.tn);
      if (st.kind == Stage::Gemm) { touched.insert(st.gemm.a_tn); touched.insert(st.gemm.b_tn); touched.insert(st.gemm.d_tn); }
      if (st.kind == Stage::Attn) { touched.insert(st.attn.q_tn); touched.insert(st.attn.k_tn); touched.insert(st.attn.v_tn); }
    }
    for (auto& t : code.prog.tnodes)
      if (t.mode == Mode::Local && touched.count(t.id)) code.local_nodes.push_back(t.id);
  }
};

}  // namespace

Code compile_program(Program prog, const CompileOptions& opt) {
  Code code;
  code.prog = std::move(prog);
  Builder b{code, opt};
  b.run();
  return code;
}

}  // namespace b200
