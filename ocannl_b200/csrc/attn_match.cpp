// Recognition of the attention chain and generation of the translation unit that instantiates the
// fused kernel (kernels/attn_sm100.cuh) with the routine's expressions.
//
// `multi_head_attention` (lib/nn_blocks.ml:222-236) with `softmax` (lib/nn_blocks.ml:137-143) lowers
// to six consecutive top-level statements:
//   1. scores[b, s, h, t] := E1( v { v := 0; for e { v := fma(q[.., s, .., e], k[.., t, .., e], v) } } )
//   2. max[b, s, h, 0]    := E2( v { v := -inf; for t { v := max(v, scores[b, s, h, t]) } } )
//   3. exp[b, s, h, t]    := E3( scores[b, s, h, t], max[b, s, h, 0] )
//   4. sum[b, s, h, 0]    := E4( v { v := 0; for t { v := v + exp[b, s, h, t] } } )
//   5. w[b, s, h, t]      := E5( exp[b, s, h, t], sum[b, s, h, 0] )
//   6. out[b, s, h, e]    := E6( v { v := 0; for t { v := fma(w[b, s, h, t], val[b, t, h, e], v) } } )
// with at most two batch symbols (b, h), 16-bit q / k / val / w of one format, a head dimension of
// 64 and 64, 128 or 256 keys.  E1 .. E6 are arbitrary expressions of the routine (a scale, a
// `where` on a mask, ...): they are emitted with the rules of every other kernel.  Operands of E1
// that run along t and vary with s (the mask) are loaded a 32 x 32 chunk at a time with whole-row
// accesses.  A node of the chain that is routine-local and not read after statement 6 is never
// written; a node the context holds is written exactly as the separate stages would write it.
#include <cmath>
#include <functional>
#include <set>
#include <sstream>

#include "compile.hpp"
#include "emit.hpp"

namespace b200 {

namespace {

struct Nest {
  std::vector<LoopDim> loops;
  const Stmt* set = nullptr;
};

bool peel(const StmtP& s, Nest* n) {
  const Stmt* b = s.get();
  while (b->kind == Stmt::For) {
    if (b->from != 0) return false;
    n->loops.push_back({b->index, b->from, b->to});
    b = b->body.get();
  }
  if (b->kind != Stmt::Set || b->vec_len > 0) return false;
  n->set = b;
  return true;
}

using Ren = std::map<std::string, std::string>;

void rename_idcs(Indices& idcs, const Ren& ren) {
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
StmtP rename_stmt(const StmtP& s, const Ren& ren);
ScalarP rename_scalar(const ScalarP& e, const Ren& ren) {
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
StmtP rename_stmt(const StmtP& s, const Ren& ren) {
  auto c = std::make_shared<Stmt>(*s);
  rename_idcs(c->idcs, ren);
  auto it = ren.find(c->index);
  if (it != ren.end()) c->index = it->second;
  for (auto& x : c->items) x = rename_stmt(x, ren);
  if (c->body) c->body = rename_stmt(c->body, ren);
  if (c->value) c->value = rename_scalar(c->value, ren);
  return c;
}

bool same_idx(const Index& a, const Index& b) { return a.kind == b.kind && a.fixed == b.fixed && a.sym == b.sym && a.terms == b.terms; }
bool same_idcs(const Indices& a, const Indices& b) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i)
    if (!same_idx(a[i], b[i])) return false;
  return true;
}

void walk(const Scalar& e, const std::function<void(const Scalar&)>& f);
void walk(const Stmt& s, const std::function<void(const Scalar&)>& f) {
  for (auto& x : s.items) walk(*x, f);
  if (s.body) walk(*s.body, f);
  if (s.value) walk(*s.value, f);
}
void walk(const Scalar& e, const std::function<void(const Scalar&)>& f) {
  f(e);
  if (e.kind == Scalar::LocalScope && e.body) walk(*e.body, f);
  for (auto& a : e.args) walk(*a.s, f);
}

// the only Local_scope of an expression (nullptr unless there is exactly one, at any depth outside other scopes)
const Scalar* single_scope(const Scalar& v) {
  const Scalar* found = nullptr;
  int n = 0;
  std::function<void(const Scalar&)> rec = [&](const Scalar& e) {
    if (e.kind == Scalar::LocalScope) { ++n; found = &e; return; }
    for (auto& a : e.args) rec(*a.s);
  };
  rec(v);
  return n == 1 ? found : nullptr;
}
bool has_scope_or_local(const Scalar& v) {
  bool any = false;
  walk(v, [&](const Scalar& e) {
    if (e.kind == Scalar::LocalScope || e.kind == Scalar::GetLocal || e.kind == Scalar::GetDyn || e.kind == Scalar::GetMerge ||
        e.kind == Scalar::EmbedIdx)
      any = true;
  });
  return any;
}

// A reduction scope:  v { v := init; for r { v := step } }  ->  the loop and the step's value
struct Reduce {
  int scope_id = 0;
  LoopDim loop;
  double init = 0;
  const Scalar* step = nullptr;
};
bool parse_reduce(const Program& P, const Scalar& sc, Reduce* out) {
  if (P.tn(sc.tn).prec != Prec::Single) return false;
  const Stmt* b = sc.body.get();
  if (b->kind != Stmt::Seq || b->items.size() != 2) return false;
  const Stmt* init = b->items[0].get();
  if (init->kind != Stmt::SetLocal || init->scope_id != sc.scope_id || init->value->kind != Scalar::Const) return false;
  const Stmt* loop = b->items[1].get();
  if (loop->kind != Stmt::For || loop->from != 0) return false;
  const Stmt* step = loop->body.get();
  if (step->kind != Stmt::SetLocal || step->scope_id != sc.scope_id) return false;
  out->scope_id = sc.scope_id;
  out->loop = {loop->index, loop->from, loop->to};
  out->init = init->value->cval;
  out->step = step->value.get();
  return true;
}
bool is_local_of(const Scalar& e, int scope_id) { return e.kind == Scalar::GetLocal && e.scope_id == scope_id; }
// fma(x, y, v) or v + x * y
bool mac_of(const Scalar& v, int scope_id, const Scalar** x, const Scalar** y) {
  if (v.kind == Scalar::Tern && v.op == "fma" && is_local_of(*v.args[2].s, scope_id)) {
    *x = v.args[0].s.get();
    *y = v.args[1].s.get();
    return true;
  }
  if (v.kind == Scalar::Bin && v.op == "add")
    for (int side = 0; side < 2; ++side) {
      const Scalar& prod = *v.args[1 - side].s;
      if (is_local_of(*v.args[side].s, scope_id) && prod.kind == Scalar::Bin && prod.op == "mul") {
        *x = prod.args[0].s.get();
        *y = prod.args[1].s.get();
        return true;
      }
    }
  return false;
}
// v op term, either order
const Scalar* combine_of(const Scalar& v, int scope_id, const char* op) {
  if (v.kind != Scalar::Bin || v.op != op) return nullptr;
  for (int side = 0; side < 2; ++side)
    if (is_local_of(*v.args[side].s, scope_id)) return v.args[1 - side].s.get();
  return nullptr;
}

bool plain_indices(const Indices& idcs) {
  for (auto& ix : idcs)
    if (ix.kind != Index::Iter && ix.kind != Index::Fixed) return false;
  return true;
}
// element stride of every symbol in a row-major node
bool strides_of(const Tnode& t, const Indices& idcs, std::map<std::string, int64_t>& stride, int64_t& const_off) {
  if (idcs.size() != t.dims.size() || !plain_indices(idcs)) return false;
  int64_t s = 1;
  const_off = 0;
  for (size_t a = idcs.size(); a-- > 0;) {
    if (idcs[a].kind == Index::Iter) stride[idcs[a].sym] += s;
    else const_off += idcs[a].fixed * s;
    s *= t.dims[a];
  }
  return true;
}
bool uses(const Indices& idcs, const std::string& sym) {
  for (auto& ix : idcs)
    if (ix.uses(sym)) return true;
  return false;
}
// maps the symbols of `read` (indices of a node whose canonical indices are `canon`) to the canonical names
bool map_through(const Indices& read, const Indices& canon, Ren* ren) {
  if (read.size() != canon.size()) return false;
  for (size_t a = 0; a < read.size(); ++a) {
    if (canon[a].kind == Index::Fixed) {
      if (!same_idx(read[a], canon[a])) return false;
    } else {
      if (read[a].kind != Index::Iter) return false;
      auto it = ren->find(read[a].sym);
      if (it != ren->end() && it->second != canon[a].sym) return false;
      (*ren)[read[a].sym] = canon[a].sym;
    }
  }
  return true;
}

const char* kB0 = "b200_b0";
const char* kB1 = "b200_b1";
const char* kS = "b200_s";
const char* kT = "b200_t";
const char* kE = "b200_e";

}  // namespace

bool match_attention(const Program& P, const std::vector<StmtP>& flat, size_t at, const CompileOptions& opt, int* n_absorbed,
                     Stage* out) {
  if (at + 6 > flat.size()) return false;
  Nest n[6];
  for (int i = 0; i < 6; ++i)
    if (!peel(flat[at + (size_t)i], &n[i])) return false;
  if (!P.statics.empty()) {
    // static indices move between launches; the fused kernel keeps to the plain case
    std::set<std::string> st;
    for (auto& s : P.statics) st.insert(s.sym);
    bool any = false;
    for (int i = 0; i < 6; ++i)
      walk(*flat[at + (size_t)i], [&](const Scalar& e) {
        for (auto& ix : e.idcs)
          for (auto& s : st)
            if (ix.uses(s)) any = true;
      });
    if (any) return false;
  }

  // ---- statement 1: scores
  const Stmt& s1 = *n[0].set;
  const Tnode& SC = P.tn(s1.tn);
  if (SC.prec != Prec::Single || SC.mode == Mode::Virtual || n[0].loops.size() < 2 || n[0].loops.size() > 4) return false;
  if (s1.idcs.size() != SC.dims.size() || s1.idcs.size() != n[0].loops.size()) return false;
  for (auto& ix : s1.idcs)
    if (ix.kind != Index::Iter) return false;
  const Scalar* sc1 = single_scope(*s1.value);
  Reduce r1;
  if (!sc1 || !parse_reduce(P, *sc1, &r1) || r1.init != 0.0) return false;
  const Scalar *x = nullptr, *y = nullptr;
  if (!mac_of(*r1.step, r1.scope_id, &x, &y)) return false;
  if (x->kind != Scalar::Get || y->kind != Scalar::Get || !plain_indices(x->idcs) || !plain_indices(y->idcs)) return false;
  const std::string t_sym = s1.idcs.back().sym;
  if (uses(x->idcs, t_sym) == uses(y->idcs, t_sym)) return false;
  if (uses(x->idcs, t_sym)) std::swap(x, y);     // x = queries, y = keys
  const Tnode &Q = P.tn(x->tn), &K = P.tn(y->tn);
  if (Q.prec != K.prec || !(Q.prec == Prec::Bfloat16 || Q.prec == Prec::Half) || Q.mode == Mode::Virtual || K.mode == Mode::Virtual)
    return false;
  std::string s_sym;
  std::vector<std::string> batch;
  for (auto& d : n[0].loops) {
    int in_lhs = 0;
    for (auto& ix : s1.idcs) in_lhs += ix.sym == d.sym;
    if (in_lhs != 1) return false;
    if (d.sym == t_sym) continue;
    const bool in_q = uses(x->idcs, d.sym), in_k = uses(y->idcs, d.sym);
    if (in_q && in_k) batch.push_back(d.sym);
    else if (in_q && !in_k && s_sym.empty()) s_sym = d.sym;
    else return false;
  }
  if (s_sym.empty() || batch.size() > 2) return false;
  auto extent_of = [](const Nest& nn, const std::string& sym) -> int64_t {
    for (auto& d : nn.loops)
      if (d.sym == sym) return d.extent();
    return -1;
  };
  const int64_t S = extent_of(n[0], s_sym), T = extent_of(n[0], t_sym), E = r1.loop.extent();
  if (E != 64 || !(T == 64 || T == 128 || T == 256) || S < 64) return false;
  if (SC.dims.back() != T) return false;
  Ren ren1;
  ren1[s_sym] = kS;
  ren1[t_sym] = kT;
  if (batch.size() == 2) { ren1[batch[0]] = kB0; ren1[batch[1]] = kB1; }
  else if (batch.size() == 1) ren1[batch[0]] = kB1;
  const int64_t B0 = batch.size() == 2 ? extent_of(n[0], batch[0]) : 1;
  const int64_t B1 = batch.size() >= 1 ? extent_of(n[0], batch.back()) : 1;
  Indices scores_idcs = s1.idcs;
  rename_idcs(scores_idcs, ren1);
  const std::string e_sym1 = r1.loop.sym;
  // extents by canonical name, for the checks on the later statements
  std::map<std::string, int64_t> role_extent = {{kS, S}, {kT, T}, {kB0, B0}, {kB1, B1}};

  // operand layouts
  struct Operand { int tn; int64_t off, row_stride, b0_stride, b1_stride; };
  auto operand = [&](const Scalar& g, const Ren& ren, const std::string& row, const std::string& unit, Operand* o) {
    Indices idcs = g.idcs;
    rename_idcs(idcs, ren);
    std::map<std::string, int64_t> st;
    int64_t off = 0;
    if (!strides_of(P.tn(g.tn), idcs, st, off)) return false;
    if (st[unit] != 1 || st[row] <= 0) return false;
    for (auto& kv : st)
      if (kv.first != unit && kv.first != row && kv.first != kB0 && kv.first != kB1 && kv.second != 0) return false;
    *o = {g.tn, off, st[row], st.count(kB0) ? st[kB0] : 0, st.count(kB1) ? st[kB1] : 0};
    // what a tensor map can express: 16-byte aligned base offset and strides
    for (int64_t v : {o->off, o->row_stride, o->b0_stride, o->b1_stride})
      if ((v * 2) % 16 != 0) return false;
    if (B0 > 1 && o->b0_stride == 0) return false;
    if (B1 > 1 && o->b1_stride == 0) return false;
    return true;
  };
  Operand oq, ok_, ov;
  {
    Ren r = ren1;
    r[e_sym1] = kE;
    if (!operand(*x, r, kS, kE, &oq) || !operand(*y, r, kT, kE, &ok_)) return false;
    if (P.tn(x->tn).dims.back() != 64 || P.tn(y->tn).dims.back() != 64) return false;
  }

  // ---- the row statements: each is mapped to the canonical symbols through its read of the node before it
  auto nest_matches = [&](const Nest& nn, const Ren& ren, bool with_t, const char* extra = nullptr) {
    std::set<std::string> seen;
    for (auto& d : nn.loops) {
      auto it = ren.find(d.sym);
      if (it == ren.end()) {
        if (d.extent() == 1) continue;
        return false;
      }
      if (extra && it->second == extra) { seen.insert(it->second); continue; }
      auto re = role_extent.find(it->second);
      if (re == role_extent.end() || re->second != d.extent()) return false;
      seen.insert(it->second);
    }
    if (seen.count(kT) != (with_t ? 1u : 0u)) return false;
    if (!seen.count(kS)) return false;
    if (B0 > 1 && !seen.count(kB0)) return false;
    if (B1 > 1 && !seen.count(kB1)) return false;
    return true;
  };
  // statement 2: row max
  const Stmt& s2 = *n[1].set;
  const Tnode& MX = P.tn(s2.tn);
  if (MX.prec != Prec::Single || MX.mode == Mode::Virtual || !plain_indices(s2.idcs)) return false;
  const Scalar* sc2 = single_scope(*s2.value);
  Reduce r2;
  if (!sc2 || !parse_reduce(P, *sc2, &r2) || !(std::isinf(r2.init) && r2.init < 0)) return false;
  const Scalar* term2 = combine_of(*r2.step, r2.scope_id, "max");
  if (!term2 || term2->kind != Scalar::Get || term2->tn != s1.tn) return false;
  Ren ren2;
  if (!map_through(term2->idcs, scores_idcs, &ren2) || ren2[r2.loop.sym] != kT || r2.loop.extent() != T) return false;
  if (!nest_matches(n[1], ren2, false)) return false;
  Indices max_idcs = s2.idcs;
  rename_idcs(max_idcs, ren2);
  if (uses(max_idcs, kT)) return false;

  // statement 3: exponentials
  const Stmt& s3 = *n[2].set;
  const Tnode& EX = P.tn(s3.tn);
  if (EX.prec != Prec::Single || EX.mode == Mode::Virtual || has_scope_or_local(*s3.value)) return false;
  Ren ren3;
  {
    bool ok = true, found = false;
    walk(*s3.value, [&](const Scalar& e) {
      if (e.kind == Scalar::Get && e.tn == s1.tn) { found = true; ok = ok && map_through(e.idcs, scores_idcs, &ren3); }
    });
    if (!ok || !found) return false;
  }
  if (!nest_matches(n[2], ren3, true)) return false;
  Indices exp_idcs = s3.idcs;
  rename_idcs(exp_idcs, ren3);
  auto row_node_ok = [&](const Tnode& t, const Indices& idcs) {
    // one row of T contiguous elements per (batch, s): t on the last axis, every other role once at most
    if (idcs.size() != t.dims.size() || idcs.empty() || idcs.back().kind != Index::Iter || idcs.back().sym != kT) return false;
    if (t.dims.back() != T) return false;
    for (size_t a = 0; a + 1 < idcs.size(); ++a)
      if (idcs[a].uses(kT) || (idcs[a].kind != Index::Iter && idcs[a].kind != Index::Fixed)) return false;
    return uses(idcs, kS);
  };
  if (!row_node_ok(SC, scores_idcs) || !row_node_ok(EX, exp_idcs)) return false;

  // statement 4: row sum
  const Stmt& s4 = *n[3].set;
  const Tnode& SM = P.tn(s4.tn);
  if (SM.prec != Prec::Single || SM.mode == Mode::Virtual || !plain_indices(s4.idcs)) return false;
  const Scalar* sc4 = single_scope(*s4.value);
  Reduce r4;
  if (!sc4 || !parse_reduce(P, *sc4, &r4) || r4.init != 0.0) return false;
  const Scalar* term4 = combine_of(*r4.step, r4.scope_id, "add");
  if (!term4 || term4->kind != Scalar::Get || term4->tn != s3.tn) return false;
  Ren ren4;
  if (!map_through(term4->idcs, exp_idcs, &ren4) || ren4[r4.loop.sym] != kT || r4.loop.extent() != T) return false;
  if (!nest_matches(n[3], ren4, false)) return false;
  Indices sum_idcs = s4.idcs;
  rename_idcs(sum_idcs, ren4);
  if (uses(sum_idcs, kT)) return false;

  // statement 5: weights
  const Stmt& s5 = *n[4].set;
  const Tnode& W = P.tn(s5.tn);
  if (!(W.prec == Prec::Bfloat16 || W.prec == Prec::Half) || W.mode == Mode::Virtual || has_scope_or_local(*s5.value)) return false;
  Ren ren5;
  {
    bool ok = true, found = false;
    walk(*s5.value, [&](const Scalar& e) {
      if (e.kind == Scalar::Get && e.tn == s3.tn) { found = true; ok = ok && map_through(e.idcs, exp_idcs, &ren5); }
    });
    if (!ok || !found) return false;
  }
  if (!nest_matches(n[4], ren5, true)) return false;
  Indices w_idcs = s5.idcs;
  rename_idcs(w_idcs, ren5);
  if (!row_node_ok(W, w_idcs)) return false;

  // statement 6: weights . values
  const Stmt& s6 = *n[5].set;
  const Tnode& O = P.tn(s6.tn);
  if (!(O.prec == Prec::Bfloat16 || O.prec == Prec::Half || O.prec == Prec::Single) || O.mode == Mode::Virtual) return false;
  const Scalar* sc6 = single_scope(*s6.value);
  Reduce r6;
  if (!sc6 || !parse_reduce(P, *sc6, &r6) || r6.init != 0.0) return false;
  const Scalar *wx = nullptr, *vy = nullptr;
  if (!mac_of(*r6.step, r6.scope_id, &wx, &vy)) return false;
  if (wx->kind != Scalar::Get || vy->kind != Scalar::Get) return false;
  if (wx->tn != s5.tn) std::swap(wx, vy);
  if (wx->tn != s5.tn || vy->tn == s5.tn) return false;
  const Tnode& V = P.tn(vy->tn);
  if (V.prec != W.prec || V.prec != Q.prec || V.mode == Mode::Virtual) return false;
  Ren ren6;
  if (!map_through(wx->idcs, w_idcs, &ren6) || ren6[r6.loop.sym] != kT || r6.loop.extent() != T) return false;
  // the one free symbol that is not a role yet is the head dimension
  std::string e_sym6;
  for (auto& d : n[5].loops)
    if (!ren6.count(d.sym) && d.extent() != 1) {
      if (!e_sym6.empty()) return false;
      e_sym6 = d.sym;
    }
  if (e_sym6.empty() || extent_of(n[5], e_sym6) != 64) return false;
  ren6[e_sym6] = kE;
  if (!nest_matches(n[5], ren6, false, kE)) return false;
  if (!operand(*vy, ren6, kT, kE, &ov) || V.dims.back() != 64) return false;
  Indices out_idcs = s6.idcs;
  rename_idcs(out_idcs, ren6);
  if (out_idcs.size() != O.dims.size() || out_idcs.empty() || out_idcs.back().kind != Index::Iter || out_idcs.back().sym != kE ||
      O.dims.back() != 64 || !plain_indices(out_idcs) || !uses(out_idcs, kS))
    return false;
  for (size_t a = 0; a + 1 < out_idcs.size(); ++a)
    if (out_idcs[a].uses(kE) || out_idcs[a].uses(kT)) return false;

  // ---- the chain's nodes are distinct, and read only in the forms matched above
  const std::vector<int> chain = {s1.tn, s2.tn, s3.tn, s4.tn, s5.tn, s6.tn};
  {
    std::set<int> uniq(chain.begin(), chain.end());
    if (uniq.size() != 6) return false;
    for (int tn : {x->tn, y->tn, vy->tn})
      if (uniq.count(tn)) return false;
  }
  struct Fwd { int tn; Indices idcs; };
  auto reads_ok = [&](const ScalarP& v, const Ren& ren, const std::vector<Fwd>& allowed) {
    ScalarP rv = rename_scalar(v, ren);
    bool ok = true;
    walk(*rv, [&](const Scalar& e) {
      if (e.kind != Scalar::Get) return;
      bool in_chain = false;
      for (int c : chain) in_chain |= e.tn == c;
      if (!in_chain) return;
      bool fine = false;
      for (auto& a : allowed) fine |= a.tn == e.tn && same_idcs(a.idcs, e.idcs);
      ok = ok && fine;
    });
    return ok;
  };
  // (inside the reductions the loop symbol is renamed to the key position, so the reads there equal the canonical ones)
  if (!reads_ok(s1.value, ren1, {}) || !reads_ok(s2.value, ren2, {{s1.tn, scores_idcs}}) ||
      !reads_ok(s3.value, ren3, {{s1.tn, scores_idcs}, {s2.tn, max_idcs}}) || !reads_ok(s4.value, ren4, {{s3.tn, exp_idcs}}) ||
      !reads_ok(s5.value, ren5, {{s3.tn, exp_idcs}, {s4.tn, sum_idcs}}) || !reads_ok(s6.value, ren6, {{s5.tn, w_idcs}}))
    return false;

  // ---- which nodes of the chain must reach memory
  auto read_later = [&](int tn) {
    bool any = false;
    for (size_t k = at + 6; k < flat.size() && !any; ++k) {
      walk(*flat[k], [&](const Scalar& e) {
        if ((e.kind == Scalar::Get || e.kind == Scalar::GetDyn) && e.tn == tn) any = true;
      });
      // a later partial write keeps the rest of the node's contents visible
      std::function<void(const Stmt&)> ws = [&](const Stmt& s) {
        if ((s.kind == Stmt::Set) && s.tn == tn) any = true;
        for (auto& x2 : s.items) ws(*x2);
        if (s.body) ws(*s.body);
      };
      ws(*flat[k]);
    }
    return any;
  };
  auto kept = [&](int tn) { return P.tn(tn).is_param() || read_later(tn); };

  // ---- generated code
  Emitter em(P);
  em.large_models = opt.large_models;
  std::ostringstream fn;
  const std::string syms =
      "  const unsigned int b200_b0 = row.b0, b200_b1 = row.b1, b200_s = row.s;\n  (void)b200_b0; (void)b200_b1; (void)b200_s;\n";
  auto zero_t = [&](Indices idcs, const char* sym) {
    for (auto& ix : idcs)
      if (ix.kind == Index::Iter && ix.sym == sym) { ix.kind = Index::Fixed; ix.fixed = 0; ix.sym.clear(); }
    return idcs;
  };
  auto row_ptr = [&](int tn, const Indices& idcs, const char* unit) {
    const Tnode& t = P.tn(tn);
    em.used_nodes.insert(tn);
    return "(unsigned long long)(" + t.ident + " + (" + em.offset(zero_t(idcs, unit), t.dims) + "))";
  };
  std::set<int> written;
  std::string rows_body;
  auto ptr_line = [&](const char* var, int tn, const Indices& idcs, const char* unit) {
    if (kept(tn)) {
      rows_body += std::string("  ") + var + " = row.ok ? " + row_ptr(tn, idcs, unit) + " : 0ull;\n";
      written.insert(tn);
    } else {
      rows_body += std::string("  ") + var + " = 0ull;\n";
    }
  };
  // (scores, exponentials and weights leave through tensor maps: kept ones are recorded, no pointer is needed)
  for (int tn : {s1.tn, s3.tn, s5.tn})
    if (kept(tn)) {
      written.insert(tn);
      em.used_nodes.insert(tn);   // stays a parameter: link checks its binding and alignment through it
    }
  ptr_line("p_max", s2.tn, max_idcs, kT);
  ptr_line("p_sum", s4.tn, sum_idcs, kT);
  ptr_line("p_out", s6.tn, out_idcs, kE);
  // the transposing stores write 16 bytes at a time
  {
    auto row16 = [&](const Tnode& t, const Indices& idcs) {
      std::map<std::string, int64_t> st;
      int64_t off = 0;
      if (!strides_of(t, idcs, st, off)) return false;
      const int eb = prec_bytes(t.prec);
      for (auto& kv : st)
        if (kv.first != kT && kv.first != kE && (kv.second * eb) % 16 != 0) return false;
      return (off * eb) % 16 == 0;
    };
    if (!row16(SC, scores_idcs) || !row16(EX, exp_idcs) || !row16(W, w_idcs) || !row16(O, out_idcs)) return false;
  }

  // E1: the score of one column.  Operands that run along t and vary with s come from register
  // tiles; those that are only ever the condition of a `where` (masks) come as one bit per element.
  std::string score_loads, score_decls, cond_rows;
  int n_cond = 0, n_tiles_used = 0;
  std::vector<int> cond_tns;
  {
    ScalarP v1 = rename_scalar(s1.value, ren1);
    // every position an operand is read at, and whether it is a `where` condition there
    struct Use { const Scalar* get; bool cond; };
    std::vector<Use> reads;
    std::function<void(const Scalar&, bool)> collect = [&](const Scalar& e, bool is_cond) {
      if (e.kind == Scalar::Get) reads.push_back({&e, is_cond});
      if (e.kind == Scalar::LocalScope) return;   // the factors of the contraction are matched inside the scope only
      for (size_t a = 0; a < e.args.size(); ++a)
        collect(*e.args[a].s, e.kind == Scalar::Tern && e.op == "where" && a == 0 && e.args[a].s->kind == Scalar::Get);
    };
    collect(*v1, false);
    int n_tiles = 0;
    for (auto& u : reads) {
      const Scalar& e = *u.get;
      if (e.idcs.empty()) continue;
      const Tnode& t = P.tn(e.tn);
      const int eb = prec_bytes(t.prec);
      if (!(eb == 4 || eb == 2) || t.prec == Prec::Fp8 || is_int_prec(t.prec) || t.mode == Mode::Virtual) continue;
      if (e.idcs.back().kind != Index::Iter || e.idcs.back().sym != kT || !plain_indices(e.idcs)) continue;
      if (!uses(e.idcs, kS)) continue;
      std::map<std::string, int64_t> st;
      int64_t off = 0;
      if (!strides_of(t, e.idcs, st, off) || st[kT] != 1) continue;
      bool aligned = (off * eb) % 16 == 0;
      for (auto& kv : st)
        if (kv.first != kT && (kv.second * eb) % 16 != 0) aligned = false;
      if (!aligned) continue;
      bool have = false;
      for (auto& lt : em.load_tiles) have = have || (lt.tn == e.tn && same_idcs(lt.idcs, e.idcs));
      if (have) continue;
      // a mask: only ever a `where` condition.  It reaches the kernel packed to one bit per element (a
      // stage of its own makes the bits); a row's bits must start on a word boundary
      bool cond_only = n_cond < 2 && st[kT] == 1 && off % 32 == 0;
      for (auto& kv : st)
        if (kv.first != kT && kv.second % 32 != 0) cond_only = false;
      for (auto& o : reads)
        if (o.get->tn == e.tn && same_idcs(o.get->idcs, e.idcs) && !o.cond) cond_only = false;
      if (cond_only) {
        // (the tile expression stands for the node's storage bits: one and zero in its format)
        const std::string one = t.prec == Prec::Single ? "1.0f : 0.0f" : t.prec == Prec::Bfloat16 ? "(unsigned short)0x3F80 : (unsigned short)0"
                                                                                                   : "(unsigned short)0x3C00 : (unsigned short)0";
        em.load_tiles.push_back({e.tn, e.idcs, "(((cw[" + std::to_string(n_cond) + "] >> b200_j) & 1u) ? " + one + ")"});
        // the row's first bit, as a byte address
        cond_rows += "  p[" + std::to_string(n_cond) + "] = row.ok ? (unsigned long long)b200_bits" + std::to_string(n_cond) + " + ((unsigned long long)(" +
                     em.offset(zero_t(e.idcs, kT), t.dims) + ") >> 3) : 0ull;\n";
        cond_tns.push_back(e.tn);
        ++n_cond;
        continue;
      }
      const std::string arr = "b200_op" + std::to_string(n_tiles++);
      em.load_tiles.push_back({e.tn, e.idcs, arr + "[b200_j]"});
      const int words = 32 * eb / 4;
      score_decls += std::string("  ") + Emitter::ctype(t.prec) + " " + arr + "[32];\n";
      score_loads += "  {\n    unsigned int b200_w[" + std::to_string(words) + "];\n    b200_attn_load_chunk<" + std::to_string(words) +
                     ">(row.stage, b200_w, row.ok ? " + row_ptr(e.tn, e.idcs, kT) + " + " + std::to_string(eb) +
                     "ull * t0 : 0ull, row.lane);\n#pragma unroll\n    for (int b200_j = 0; b200_j < 32; ++b200_j) " + arr + "[b200_j] = " +
                     (eb == 4 ? "__uint_as_float(b200_w[b200_j])" : "(unsigned short)(b200_w[b200_j >> 1] >> (16 * (b200_j & 1)))") +
                     ";\n  }\n";
    }
    n_tiles_used = n_tiles;
    em.scope_subst[r1.scope_id] = "b200_acc";
    const int reads_before = em.direct_reads;
    Emitter::Res r = em.scalar(Prec::Single, *v1);
    if (!r.defs.empty()) return false;
    // rows beyond the last query compute on whatever the registers hold (nothing of it is stored)
    // unless the expression reads memory itself: no branch per element
    const std::string guard1 = em.direct_reads > reads_before ? "row.ok ? (float)(" + r.expr + ") : 0.f" : "(float)(" + r.expr + ")";
    fn << "__device__ __forceinline__ void b200_attn_score_chunk(const b200_attn_row& row, unsigned int t0, const unsigned int* acc, float* x, "
          "const unsigned int* cw B200_ATTN_PARAMS) {\n"
       << syms << score_decls << score_loads
       << "#pragma unroll\n  for (int b200_j = 0; b200_j < 32; ++b200_j) {\n    const unsigned int b200_t = t0 + (unsigned int)b200_j; (void)b200_t;\n"
       << "    const float b200_acc = __uint_as_float(acc[b200_j]);\n"
       << "    x[b200_j] = " << guard1 << ";\n  }\n}\n";
    fn << "__device__ __forceinline__ void b200_attn_cond_rows(const b200_attn_row& row, unsigned long long* p B200_ATTN_PARAMS) {\n"
       << syms << cond_rows << "}\n";
    em.scope_subst.clear();
    em.load_tiles.clear();
  }
  // E2 / E4: what is stored from the reduced value
  {
    ScalarP v2 = rename_scalar(s2.value, ren2);
    em.scope_subst[r2.scope_id] = "reduced";
    Emitter::Res r = em.scalar(Prec::Single, *v2);
    if (!r.defs.empty()) return false;
    fn << "__device__ __forceinline__ float b200_attn_max_init() { return " << em.constant(r2.init, Prec::Single) << "; }\n"
       << "__device__ __forceinline__ float b200_attn_row_max(const b200_attn_row& row, float reduced B200_ATTN_PARAMS) {\n"
       << syms << "  return row.ok ? (float)(" << r.expr << ") : 0.f;\n}\n";
    em.scope_subst.clear();
    ScalarP v4 = rename_scalar(s4.value, ren4);
    em.scope_subst[r4.scope_id] = "reduced";
    Emitter::Res q = em.scalar(Prec::Single, *v4);
    if (!q.defs.empty()) return false;
    fn << "__device__ __forceinline__ float b200_attn_row_sum(const b200_attn_row& row, float reduced B200_ATTN_PARAMS) {\n"
       << syms << "  return row.ok ? (float)(" << q.expr << ") : 1.f;\n}\n";
    em.scope_subst.clear();
  }
  // E3
  {
    ScalarP v3 = rename_scalar(s3.value, ren3);
    em.forwarded[s1.tn] = {scores_idcs, "x[b200_j]"};
    em.forwarded[s2.tn] = {max_idcs, "mx"};
    const int reads_before = em.direct_reads;
    Emitter::Res r = em.scalar(Prec::Single, *v3);
    if (!r.defs.empty()) return false;
    const std::string guard3 = em.direct_reads > reads_before ? "row.ok ? (float)(" + r.expr + ") : 0.f" : "(float)(" + r.expr + ")";
    fn << "__device__ __forceinline__ void b200_attn_exp_chunk(const b200_attn_row& row, unsigned int t0, float* x, float mx B200_ATTN_PARAMS) {\n"
       << syms
       << "#pragma unroll\n  for (int b200_j = 0; b200_j < 32; ++b200_j) {\n    const unsigned int b200_t = t0 + (unsigned int)b200_j; (void)b200_t;\n"
       << "    x[b200_j] = " << guard3 << ";\n  }\n}\n";
    em.forwarded.clear();
  }
  // E5: the weights as rounded values, packed two to a word.  When the expression divides by a
  // value that is the same for the whole row (the sum), the divisor is prepared once per row.
  {
    ScalarP v5 = rename_scalar(s5.value, ren5);
    em.forwarded[s3.tn] = {exp_idcs, "e[b200_j]"};
    em.forwarded[s4.tn] = {sum_idcs, "sum"};
    // the expression twice when it divides by a row-invariant value: with the prepared divisor's
    // short sequence, and with the plain division for divisors outside its range (one test per chunk)
    std::string divisor_def, fast_expr;
    const int reads_before = em.direct_reads;
    if (v5->kind == Scalar::Bin && v5->op == "div" && (W.prec == Prec::Bfloat16 || W.prec == Prec::Half)) {
      bool row_invariant = true;
      walk(*v5->args[1].s, [&](const Scalar& e) {
        if (e.kind == Scalar::Get && e.tn != s4.tn && uses(e.idcs, kT)) row_invariant = false;
        if (e.kind == Scalar::Get && e.tn == s3.tn) row_invariant = false;
        if (e.kind == Scalar::EmbedIdx && e.idx.uses(kT)) row_invariant = false;
      });
      Emitter::Res d = em.scalar(W.prec, *v5->args[1].s);
      if (row_invariant && d.defs.empty() && d.expr.find("b200_j") == std::string::npos && d.expr.find("b200_t") == std::string::npos) {
        em.divisor_vars[d.expr] = "b200_dv";
        divisor_def = "  const b200_divisor b200_dv = b200_divisor_of(" + d.expr + ");\n";
        Emitter::Res f = em.scalar(W.prec, *v5);
        if (!f.defs.empty()) return false;
        fast_expr = f.expr;
        em.divisor_vars.clear();
      }
    }
    Emitter::Res r = em.scalar(W.prec, *v5);
    if (!r.defs.empty()) return false;
    const bool guarded = em.direct_reads > reads_before;
    auto loop = [&](const std::string& expr) {
      return "#pragma unroll\n  for (int b200_j = 0; b200_j < 32; ++b200_j) {\n    const unsigned int b200_t = t0 + (unsigned int)b200_j; (void)b200_t;\n"
             "    b200_a[b200_j] = " + (guarded ? "row.ok ? (float)(" + expr + ") : 0.f" : "(float)(" + expr + ")") + ";\n  }\n";
    };
    const char* pack = W.prec == Prec::Bfloat16 ? "b200_pack_bf" : "b200_pack_hf";
    fn << "__device__ __forceinline__ void b200_attn_weight_chunk(const b200_attn_row& row, unsigned int t0, const float* e, float sum, unsigned int* w B200_ATTN_PARAMS) {\n"
       << syms << divisor_def << "  float b200_a[32];\n";
    if (!fast_expr.empty()) fn << "  if (b200_dv.fast) {\n" << loop(fast_expr) << "  } else {\n" << loop(r.expr) << "  }\n";
    else fn << loop(r.expr);
    fn << "#pragma unroll\n  for (int b200_j = 0; b200_j < 16; ++b200_j) w[b200_j] = " << pack << "(b200_a[2 * b200_j], b200_a[2 * b200_j + 1]);\n}\n";
    em.forwarded.clear();
    em.divisor_vars.clear();
  }
  // E6
  {
    ScalarP v6 = rename_scalar(s6.value, ren6);
    em.scope_subst[r6.scope_id] = "b200_acc";
    Emitter::Res r = em.scalar(O.prec, *v6);
    if (!r.defs.empty()) return false;
    fn << "__device__ __forceinline__ void b200_attn_out_chunk(const b200_attn_row& row, unsigned int e0, const unsigned int* acc, unsigned int* w B200_ATTN_PARAMS) {\n"
       << syms << "  float b200_a[32];\n"
       << "#pragma unroll\n  for (int b200_j = 0; b200_j < 32; ++b200_j) {\n    const unsigned int b200_e = e0 + (unsigned int)b200_j; (void)b200_e;\n"
       << "    const float b200_acc = __uint_as_float(acc[b200_j]);\n"
       << "    b200_a[b200_j] = row.ok ? (float)(" << r.expr << ") : 0.f;\n  }\n";
    if (O.prec == Prec::Single)
      fn << "#pragma unroll\n  for (int b200_j = 0; b200_j < 32; ++b200_j) w[b200_j] = __float_as_uint(b200_a[b200_j]);\n}\n";
    else
      fn << "#pragma unroll\n  for (int b200_j = 0; b200_j < 16; ++b200_j) w[b200_j] = "
         << (O.prec == Prec::Bfloat16 ? "b200_pack_bf" : "b200_pack_hf") << "(b200_a[2 * b200_j], b200_a[2 * b200_j + 1]);\n}\n";
    em.scope_subst.clear();
  }
  fn << "__device__ __forceinline__ void b200_attn_rows(const b200_attn_row& row, unsigned long long& p_max, unsigned long long& p_sum, "
        "unsigned long long& p_out B200_ATTN_PARAMS) {\n"
     << syms << rows_body << "}\n";
  if (em.uses_merge || em.uses_statics) return false;

  // parameters: every node the generated code names
  std::string params, args;
  std::vector<KArg> kargs;
  for (auto& t : P.tnodes) {
    if (!em.used_nodes.count(t.id) || t.mode == Mode::Virtual) continue;
    const bool w = written.count(t.id) > 0;
    params += std::string(", ") + (w ? "" : "const ") + Emitter::ctype(t.prec) + "* " + (w ? "" : "__restrict__ ") + t.ident;
    args += ", " + t.ident;
    kargs.push_back({KArg::Node, t.id});
  }
  for (int c = 0; c < n_cond; ++c) {
    params += ", const unsigned char* __restrict__ b200_bits" + std::to_string(c);
    args += ", b200_bits" + std::to_string(c);
    kargs.push_back({KArg::Scratch, 0});   // the planner assigns the offset of the packed bits
  }

  Stage st;
  st.kind = Stage::Attn;
  st.args = kargs;
  st.epi_params = params;
  st.epi_args = args;
  st.block = 256;
  st.min_align = 16;
  AttnPlan& a = st.attn;
  a.q_tn = oq.tn; a.k_tn = ok_.tn; a.v_tn = ov.tn;
  a.q_off = oq.off; a.k_off = ok_.off; a.v_off = ov.off;
  a.S = S; a.T = T; a.E = E; a.B0 = B0; a.B1 = B1;
  a.q_row = oq.row_stride; a.k_row = ok_.row_stride; a.v_row = ov.row_stride;
  a.q_b0 = oq.b0_stride; a.q_b1 = oq.b1_stride;
  a.k_b0 = ok_.b0_stride; a.k_b1 = ok_.b1_stride;
  a.v_b0 = ov.b0_stride; a.v_b1 = ov.b1_stride;
  a.in_prec = Q.prec;
  a.out_bytes = prec_bytes(O.prec);
  a.n_cond = n_cond;
  a.cond_tns = cond_tns;
  a.n_tiles = n_tiles_used;
  {
    auto fill = [&](AttnPlan::RowNode& rn, int tn, const Indices& idcs) {
      std::map<std::string, int64_t> stx;
      int64_t off = 0;
      strides_of(P.tn(tn), idcs, stx, off);
      rn.keep = written.count(tn) > 0;
      rn.tn = tn;
      rn.off = off;
      rn.row = stx[kS];
      rn.b0 = stx.count(kB0) ? stx[kB0] : 0;
      rn.b1 = stx.count(kB1) ? stx[kB1] : 0;
    };
    fill(a.scores, s1.tn, scores_idcs);
    fill(a.exps, s3.tn, exp_idcs);
    fill(a.weights, s5.tn, w_idcs);
  }
  a.code = fn.str();
  for (int c : chain)
    if (written.count(c)) st.writes.push_back(c);
  int kept_rows = 0;
  for (int c : {s1.tn, s3.tn, s5.tn}) kept_rows += written.count(c) > 0;
  st.note = "fused attention: scores, softmax and weights . values in one tcgen05 kernel (" + std::to_string(T) + " keys, " +
            std::to_string(kept_rows) + " of the 3 row nodes written)";
  *out = st;
  *n_absorbed = 6;
  return true;
}

std::string attn_translation_unit(const Program&, Stage& st, const std::string& kernel_name) {
  const AttnPlan& a = st.attn;
  const unsigned int fmt = a.in_prec == Prec::Bfloat16 ? 1u : 0u;
  // instruction descriptors: fp32 accumulate, operand formats, majors (bit 16: B is n-major), N >> 3, M >> 4
  const unsigned int idesc1 = (1u << 4) | (fmt << 7) | (fmt << 10) | ((unsigned int)(a.T >> 3) << 17) | ((128u >> 4) << 24);
  const unsigned int idesc2 = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((unsigned int)(a.E >> 3) << 17) | ((128u >> 4) << 24);
  std::ostringstream o;
  o << kNumericsSource << "\n#define B200_ELEM_BYTES 2\n#define B200_CTA_PAIR 0\n" << kTcSource << "\n";
  o << "#define B200_ATTN_NAME " << kernel_name << "\n#define B200_T " << a.T << "\n#define B200_E " << a.E << "\n#define B200_IDESC1 "
    << idesc1 << "u\n#define B200_IDESC2 " << idesc2 << "u\n#define B200_HALF " << (a.in_prec == Prec::Half ? 1 : 0)
    << "\n#define B200_OUT_BYTES " << a.out_bytes << "\n#define B200_ATTN_NCOND " << a.n_cond << "\n#define B200_ATTN_NTILES " << a.n_tiles
    << "\n#define B200_KEEP_SCORES " << (a.scores.keep ? 1 : 0) << "\n#define B200_KEEP_EXP " << (a.exps.keep ? 1 : 0)
    << "\n#define B200_KEEP_W " << (a.weights.keep ? 1 : 0) << "\n#define B200_ATTN_PARAMS " << st.epi_params << "\n#define B200_ATTN_ARGS "
    << st.epi_args << "\n";
  o << kAttnSource << "\n" << a.code << "\n";
  const int64_t ra0 = 128 * a.E * 2 + a.T * a.E * 2, p = 128 * a.T * 2;
  const int64_t region_a = std::max<int64_t>(std::max(ra0, p), 8 * 4096);
  st.smem_bytes = (int)(region_a + a.T * a.E * 2 + 1024 + 64 + 1024);
  return o.str();
}

}  // namespace b200
