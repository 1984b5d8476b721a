// Recognition of dense contractions in a loop nest and generation of the translation unit
// that instantiates the tcgen05 kernel (kernels/gemm_sm100.cuh) with the routine's epilogue.
//
// Two shapes are recognised (they are what `Assignments.to_low_level` + inlining produce for
// `+*`/matmul, arrayjit/lib/assignments.ml:311-488, arrayjit/lib/low_level.ml:750-1150,1631-1634):
//   A. virtual accumulator inside the consumer:
//        for f.. { t[f..] := E( v { v := 0; for k.. { v := fma(x[..], y[..], v) } } ) }
//   B. materialised accumulate:
//        [zero_out t;] for f.., k.. { t[f..] := fma(x[..], y[..], t[f..]) }
// A loop symbol is a batch axis when both operands carry it, an M (N) axis when only the
// first (second) operand carries it, and a K axis when it is reduced.  Operands are bf16 or
// half pairs, or single-precision pairs that the tensor cores read as tf32 (`tf32=0` keeps those
// on the exact generic path).  Anything else —
// affine or static indices in the operands, mixed operand precisions, an accumulator that
// is not fp32 (the cc backend would round every step, arrayjit/lib/cc_backend.ml:169-186),
// strides the tensor maps cannot express — is left to the generic loop-nest kernels.
#include <algorithm>
#include <cstdlib>
#include <functional>
#include <set>
#include <sstream>

#include "compile.hpp"
#include "emit.hpp"

namespace b200 {

namespace {

const int kAccScope = -777;  // pseudo scope id standing for the TMEM accumulator value

struct SymInfo {
  std::string sym;
  int64_t extent = 1;
  int64_t sa = 0, sb = 0, sd = 0;
  bool in_a = false, in_b = false, in_d = false;
};

// element stride of `sym` in a row-major tensor indexed by idcs; false on unsupported index forms
bool strides_of(const Tnode& t, const Indices& idcs, std::map<std::string, int64_t>& stride, int64_t& const_off) {
  if (idcs.size() != t.dims.size()) return false;
  int64_t s = 1;
  const_off = 0;
  for (size_t a = idcs.size(); a-- > 0;) {
    const Index& ix = idcs[a];
    if (ix.kind == Index::Iter) stride[ix.sym] += s;
    else if (ix.kind == Index::Fixed) const_off += ix.fixed * s;
    else return false;
    s *= t.dims[a];
  }
  return true;
}

bool is_get_of(const Scalar& e, int tn, const Indices& idcs) {
  if (e.kind != Scalar::Get || e.tn != tn || e.idcs.size() != idcs.size()) return false;
  for (size_t i = 0; i < idcs.size(); ++i) {
    const Index &a = e.idcs[i], &b = idcs[i];
    if (a.kind != b.kind || a.fixed != b.fixed || a.sym != b.sym || a.terms != b.terms) return false;
  }
  return true;
}

// the multiply-accumulate step: returns the two factors
bool mac_step(const Scalar& v, const std::function<bool(const Scalar&)>& is_acc, const Scalar** x, const Scalar** y) {
  if (v.kind == Scalar::Tern && v.op == "fma" && is_acc(*v.args[2].s)) {
    *x = v.args[0].s.get();
    *y = v.args[1].s.get();
    return true;
  }
  if (v.kind == Scalar::Bin && v.op == "add") {
    for (int side = 0; side < 2; ++side) {
      const Scalar& acc = *v.args[side].s;
      const Scalar& prod = *v.args[1 - side].s;
      if (is_acc(acc) && prod.kind == Scalar::Bin && prod.op == "mul") {
        *x = prod.args[0].s.get();
        *y = prod.args[1].s.get();
        return true;
      }
    }
  }
  return false;
}

void walk_stmt_simple(const Stmt& s, const std::function<void(const Scalar&)>& f);
void walk_scalar_simple(const Scalar& e, const std::function<void(const Scalar&)>& f) {
  f(e);
  if (e.kind == Scalar::LocalScope) walk_stmt_simple(*e.body, f);
  for (auto& a : e.args) walk_scalar_simple(*a.s, f);
}
void walk_stmt_simple(const Stmt& s, const std::function<void(const Scalar&)>& f) {
  for (auto& x : s.items) walk_stmt_simple(*x, f);
  if (s.body) walk_stmt_simple(*s.body, f);
  if (s.value) walk_scalar_simple(*s.value, f);
}

}  // namespace

static void gemm_tile_shape(const GemmPlan& g, int* bn_out, bool* pair_out);
static bool match_gemm_mode(const Program& P, const std::vector<LoopDim>& nest, const Stmt& set, bool zeroed_before,
                            const CompileOptions& opt, const std::vector<Follower>& followers, int* n_fused, Stage* out,
                            bool pair);
static int gemm_split_k(const GemmPlan& g);

// The epilogue is first tried over pairs of columns (packed 16-bit arithmetic); anything that form
// cannot express falls back to one column at a time.
bool match_gemm(const Program& P, const std::vector<LoopDim>& nest, const Stmt& set, bool zeroed_before,
                const CompileOptions& opt, const std::vector<Follower>& followers, int* n_fused, Stage* out) {
  if (opt.enable_pairs) {
    Stage trial = *out;
    int fused_pair = 0;
    bool ok = false;
    try {
      ok = match_gemm_mode(P, nest, set, zeroed_before, opt, followers, &fused_pair, &trial, true);
    } catch (const Error&) {
    }
    if (ok) {
      // the one-column form is preferred when it can take whole-row assignments into the epilogue
      Stage plain = *out;
      int fused_plain = 0;
      bool ok_plain = false;
      try {
        ok_plain = match_gemm_mode(P, nest, set, zeroed_before, opt, followers, &fused_plain, &plain, false);
      } catch (const Error&) {
      }
      if (ok_plain && plain.row_followers > 0 && fused_plain > fused_pair) {
        *out = plain;
        *n_fused = fused_plain;
      } else {
        *out = trial;
        *n_fused = fused_pair;
      }
      return true;
    }
  }
  return match_gemm_mode(P, nest, set, zeroed_before, opt, followers, n_fused, out, false);
}

static bool match_gemm_mode(const Program& P, const std::vector<LoopDim>& nest, const Stmt& set, bool zeroed_before,
                            const CompileOptions& opt, const std::vector<Follower>& followers, int* n_fused, Stage* out,
                            const bool pair) {
  *n_fused = 0;
  if (set.kind != Stmt::Set || set.vec_len > 0) return false;
  const Tnode& D = P.tn(set.tn);
  std::set<std::string> statics;
  for (auto& s : P.statics) statics.insert(s.sym);

  const Scalar *x = nullptr, *y = nullptr;
  std::vector<LoopDim> red;  // reduction loops, outer to inner
  std::vector<LoopDim> free_loops;
  const Scalar* scope = nullptr;
  bool form_b = false;

  // ---- form B
  {
    const Scalar& v = *set.value;
    auto is_acc = [&](const Scalar& e) { return is_get_of(e, set.tn, set.idcs); };
    if (mac_step(v, is_acc, &x, &y)) {
      form_b = true;
      for (auto& d : nest) {
        bool in_lhs = false;
        for (auto& ix : set.idcs)
          if (ix.uses(d.sym)) in_lhs = true;
        (in_lhs ? free_loops : red).push_back(d);
      }
      if (D.prec != Prec::Single) return false;  // accumulating in a rounded type: not a tensor-core job
    }
  }
  // ---- form A
  if (!form_b) {
    int n_scopes = 0;
    std::function<void(const Scalar&)> find = [&](const Scalar& e) {
      if (e.kind == Scalar::LocalScope) {
        ++n_scopes;
        scope = &e;
        return;
      }
      for (auto& a : e.args) find(*a.s);
    };
    find(*set.value);
    if (n_scopes != 1) return false;
    if (P.tn(scope->tn).prec != Prec::Single) return false;
    const Stmt* b = scope->body.get();
    if (b->kind == Stmt::Seq) {
      if (b->items.size() != 2 || b->items[0]->kind != Stmt::SetLocal || b->items[0]->scope_id != scope->scope_id ||
          b->items[0]->value->kind != Scalar::Const || b->items[0]->value->cval != 0.0)
        return false;
      b = b->items[1].get();
    }
    while (b->kind == Stmt::For) {
      red.push_back({b->index, b->from, b->to});
      b = b->body.get();
    }
    if (b->kind != Stmt::SetLocal || b->scope_id != scope->scope_id) return false;
    auto is_acc = [&](const Scalar& e) { return e.kind == Scalar::GetLocal && e.scope_id == scope->scope_id; };
    if (!mac_step(*b->value, is_acc, &x, &y)) return false;
    free_loops = nest;
    // no other use of the accumulator's local inside the expression
    int uses = 0;
    std::function<void(const Scalar&)> cnt = [&](const Scalar& e) {
      if (e.kind == Scalar::GetLocal && e.scope_id == scope->scope_id) ++uses;
      if (e.kind == Scalar::LocalScope) return;
      for (auto& a : e.args) cnt(*a.s);
    };
    cnt(*set.value);
    if (uses) return false;
  }
  if (red.empty() || free_loops.empty()) return false;
  for (auto& d : nest)
    if (d.from != 0) return false;
  for (auto& d : red)
    if (d.from != 0) return false;
  if (x->kind != Scalar::Get || y->kind != Scalar::Get) return false;
  const Tnode &X = P.tn(x->tn), &Y = P.tn(y->tn);
  if (X.prec != Y.prec) return false;
  // bf16 / half operands (kind::f16) or, unless switched off, single-precision operands read as tf32
  // (kind::tf32: the tensor cores use the upper 19 bits of each operand, products are summed in fp32)
  if (!(X.prec == Prec::Bfloat16 || X.prec == Prec::Half || (X.prec == Prec::Single && opt.enable_tf32))) return false;
  if (X.mode == Mode::Virtual || Y.mode == Mode::Virtual) return false;

  // ---- strides
  std::map<std::string, int64_t> sx, sy, sd;
  int64_t offx = 0, offy = 0, offd = 0;
  if (!strides_of(X, x->idcs, sx, offx) || !strides_of(Y, y->idcs, sy, offy) || !strides_of(D, set.idcs, sd, offd))
    return false;
  for (auto& m : {sx, sy})
    for (auto& kv : m)
      if (statics.count(kv.first)) return false;
  // every free symbol indexes the output exactly once; reduction symbols never do
  std::vector<SymInfo> F, R;
  std::set<std::string> known;
  for (auto& d : free_loops) {
    SymInfo s{d.sym, d.extent(), sx.count(d.sym) ? sx[d.sym] : 0, sy.count(d.sym) ? sy[d.sym] : 0,
              sd.count(d.sym) ? sd[d.sym] : 0};
    s.in_a = sx.count(d.sym);
    s.in_b = sy.count(d.sym);
    s.in_d = sd.count(d.sym);
    if (!s.in_d) return false;
    int occurrences = 0;
    for (auto& ix : set.idcs)
      if (ix.kind == Index::Iter && ix.sym == d.sym) ++occurrences;
    if (occurrences != 1) return false;
    if (!s.in_a && !s.in_b) return false;
    if (s.extent <= 0) return false;
    F.push_back(s);
    known.insert(d.sym);
  }
  for (auto& d : red) {
    SymInfo s{d.sym, d.extent(), sx.count(d.sym) ? sx[d.sym] : 0, sy.count(d.sym) ? sy[d.sym] : 0, 0};
    s.in_a = sx.count(d.sym);
    s.in_b = sy.count(d.sym);
    if (!s.in_a || !s.in_b || sd.count(d.sym)) return false;
    R.push_back(s);
    known.insert(d.sym);
  }
  for (auto& m : {sx, sy, sd})
    for (auto& kv : m)
      if (!known.count(kv.first) && !statics.count(kv.first)) return false;
  for (auto& kv : sd)
    if (statics.count(kv.first)) { /* a static slice of the output moves with each launch: fine, the epilogue indexes it */ }

  // ---- which operand sits on the N side: the output's unit-stride symbol should be N
  bool swap = false;
  for (auto& s : F)
    if (s.sd == 1 && s.extent > 1 && s.in_a && !s.in_b) swap = true;
  if (swap) {
    std::swap(x, y);
    for (auto& s : F) { std::swap(s.sa, s.sb); std::swap(s.in_a, s.in_b); }
    for (auto& s : R) { std::swap(s.sa, s.sb); std::swap(s.in_a, s.in_b); }
    std::swap(offx, offy);
  }
  const Tnode &A = P.tn(x->tn), &B = P.tn(y->tn);

  // ---- group and merge symbols
  struct Dim {
    std::vector<std::pair<std::string, int64_t>> syms;  // (symbol, extent), outer to inner
    int64_t extent = 1, sa = 0, sb = 0, sd = 0;
  };
  auto merge = [](std::vector<Dim>& g) {
    for (size_t i = 0; i + 1 < g.size();) {
      Dim &o = g[i], &n = g[i + 1];
      bool ok = o.sa == n.extent * n.sa && o.sb == n.extent * n.sb && o.sd == n.extent * n.sd;
      if (ok) {
        Dim m = n;
        m.extent = o.extent * n.extent;
        m.syms.insert(m.syms.begin(), o.syms.begin(), o.syms.end());
        g[i] = m;
        g.erase(g.begin() + i + 1);
      } else {
        ++i;
      }
    }
  };
  std::vector<Dim> gm, gn, gk, gb;
  for (auto& s : F) {
    if (s.extent == 1) continue;  // degenerate loop: contributes nothing to addressing
    Dim d{{{s.sym, s.extent}}, s.extent, s.sa, s.sb, s.sd};
    if (s.in_a && s.in_b) gb.push_back(d);
    else if (s.in_a) gm.push_back(d);
    else gn.push_back(d);
  }
  for (auto& s : R) {
    if (s.extent == 1) continue;
    gk.push_back(Dim{{{s.sym, s.extent}}, s.extent, s.sa, s.sb, 0});
  }
  merge(gm); merge(gn); merge(gk); merge(gb);
  // leftover outer M / N dims become batch axes along which one operand is broadcast
  while (gm.size() > 1) { gb.push_back(gm.front()); gm.erase(gm.begin()); }
  while (gn.size() > 1) { gb.push_back(gn.front()); gn.erase(gn.begin()); }
  if (gm.size() != 1 || gn.size() != 1 || gk.size() != 1 || gb.size() > 2) return false;
  const Dim &dm = gm[0], &dn = gn[0], &dk = gk[0];

  GemmPlan g;
  g.a_tn = x->tn;
  g.b_tn = y->tn;
  g.d_tn = set.tn;
  g.m = {dm.extent, dm.sa, 0, dm.sd};
  g.n = {dn.extent, 0, dn.sb, dn.sd};
  g.k = {dk.extent, dk.sa, dk.sb, 0};
  for (auto& d : gb) g.batch.push_back({d.extent, d.sa, d.sb, d.sd});
  g.a_off = offx;
  g.b_off = offy;
  g.in_prec = A.prec;
  g.accumulate = form_b && !zeroed_before;
  if (g.k.sa == 1) g.a_kmajor = true;
  else if (g.m.sa == 1) g.a_kmajor = false;
  else return false;
  if (g.k.sb == 1) g.b_kmajor = true;
  else if (g.n.sb == 1) g.b_kmajor = false;
  else return false;

  // ---- what the tensor maps can express: 16-byte aligned bases and strides, 32-bit extents
  const int eb = prec_bytes(A.prec);
  auto ok16 = [&](int64_t elems) { return (elems * eb) % 16 == 0; };
  if (!ok16(g.a_off) || !ok16(g.b_off)) return false;
  if (!ok16(g.a_kmajor ? g.m.sa : g.k.sa) || !ok16(g.b_kmajor ? g.n.sb : g.k.sb)) return false;
  for (auto& b : g.batch)
    if ((b.sa && !ok16(b.sa)) || (b.sb && !ok16(b.sb))) return false;
  if (g.m.extent >= (1ll << 31) || g.n.extent >= (1ll << 31) || g.k.extent >= (1ll << 31)) return false;
  // ---- worth a tensor-core launch?
  if (g.m.extent < 32 || g.n.extent < 8 || g.k.extent < 16 || g.flops() < 4.0e6) return false;
  (void)B;
  (void)opt;

  // ---- epilogue: recover the loop symbols from (batch, m, n) and run the consumer assignment
  Emitter em(P);
  em.large_models = opt.large_models;
  std::ostringstream ep;
  auto recover = [&](const Dim& d, const std::string& var) {
    std::string rem = var;
    for (size_t i = d.syms.size(); i-- > 0;) {
      const auto& s = d.syms[i];
      if (i == 0) ep << "    const unsigned int " << s.first << " = " << rem << ";\n";
      else {
        ep << "    const unsigned int " << s.first << " = " << rem << " % " << s.second << "u;\n";
        std::string nr = "b200_q_" + s.first;
        ep << "    const unsigned int " << nr << " = " << rem << " / " << s.second << "u;\n";
        rem = nr;
      }
    }
  };
  // degenerate (extent 1) free loops and unit reductions still name symbols the epilogue may use
  std::string unit_syms;
  for (auto& s : F)
    if (s.extent == 1) unit_syms += "    const unsigned int " + s.sym + " = 0u;\n";

  // Every node the epilogue writes goes through a per-thread register tile (one value per
  // column of the chunk) so that the tile can be stored with 16-byte vector stores, and so
  // that fused follow-up assignments read the producer's value from registers.
  struct Out {
    int tn;
    Indices idcs;
    std::string arr;
    bool unit_n = false;   // the node's last axis is the n symbol: a chunk is contiguous
    std::string row_off;   // element offset of column n = 0 of this row
    int tma = -1;          // index of the tensor map that stores this node's chunks (-1: none)
  };
  std::vector<Out> outs;
  // The n axis may be several merged loop symbols (the (head, d) of an attention projection).  A
  // node runs "along n" when its trailing axes are exactly those symbols, in order, over axes as
  // long as the symbols' loops (the outermost may be longer): column n of a row then lies n
  // elements after column 0.  `along_n` returns the indices of column 0, or nothing.
  const size_t n_syms = dn.syms.size();
  const std::string n_sym = n_syms >= 1 ? dn.syms.back().first : std::string();   // innermost: neighbours differ in it
  auto along_n = [&](const Indices& idcs, const std::vector<int64_t>& dims, Indices* row) {
    if (n_syms == 0 || idcs.size() < n_syms || idcs.size() != dims.size()) return false;
    const size_t first = idcs.size() - n_syms;
    for (size_t q = 0; q < n_syms; ++q) {
      const Index& ix = idcs[first + q];
      if (ix.kind != Index::Iter || ix.sym != dn.syms[q].first) return false;
      if (q > 0 && dims[first + q] != dn.syms[q].second) return false;
    }
    for (size_t a = 0; a < first; ++a)
      for (auto& sy : dn.syms)
        if (idcs[a].uses(sy.first)) return false;
    *row = idcs;
    for (size_t q = 0; q < n_syms; ++q) {
      Index& ix = (*row)[first + q];
      ix.kind = Index::Fixed;
      ix.fixed = 0;
      ix.sym.clear();
    }
    return true;
  };
  // pair mode: b200_j counts PAIRS of columns; tiles hold one pair per entry.  Neighbouring columns
  // differ only in the innermost n symbol as long as its loop has an even length.
  // (a materialised accumulate that reads its output back stays in the one-column form)
  if (pair && ((form_b && g.accumulate) || n_sym.empty() || g.n.extent % 2 != 0 || dn.syms.back().second % 2 != 0)) return false;
  em.pair = pair;
  em.pair_sym = n_sym;
  bool pair_fail = false;
  auto add_out = [&](int tn, const Indices& idcs) {
    Out o;
    o.tn = tn;
    o.idcs = idcs;
    o.arr = "b200_o" + std::to_string(tn);
    const Tnode& t = P.tn(tn);
    {
      Indices row;
      if (along_n(idcs, t.dims, &row)) {
        o.unit_n = true;
        o.row_off = em.offset(row, t.dims);
      }
    }
    if (pair && (!o.unit_n || !Emitter::pair_prec(t.prec))) pair_fail = true;
    em.set_redirect[tn] = {idcs, o.arr + "[b200_j]"};
    em.used_nodes.insert(tn);
    outs.push_back(o);
  };

  // A node as a regular [batch.., m, n] array for this contraction, for the TMA unit: the m symbols
  // (and each batch group's) compose to one stride, n is contiguous, everything 16-byte aligned,
  // and no other symbol moves the address.
  auto make_map = [&](int tn, const Indices& idcs, OutMap* m) {
    const Tnode& t = P.tn(tn);
    const int ebytes = prec_bytes(t.prec);
    std::map<std::string, int64_t> st_;
    int64_t off = 0;
    if (!strides_of(t, idcs, st_, off)) return false;
    auto group_stride = [&](const Dim& d, int64_t* stride) {
      // outer to inner: each symbol's stride is the next one's stride times its extent
      int64_t inner = -1;
      for (size_t i = d.syms.size(); i-- > 0;) {
        const int64_t s_ = st_.count(d.syms[i].first) ? st_[d.syms[i].first] : 0;
        if (i + 1 == d.syms.size()) inner = s_;
        else if (s_ != st_[d.syms[i + 1].first] * d.syms[i + 1].second) return false;
      }
      *stride = inner;
      return inner > 0;
    };
    m->tn = tn;
    m->off = off;
    int64_t n_stride = 0;
    if (!group_stride(dm, &m->m_stride) || !group_stride(dn, &n_stride) || n_stride != 1) return false;
    if (gb.size() == 2) { if (!group_stride(gb[0], &m->b0_stride) || !group_stride(gb[1], &m->b1_stride)) return false; }
    else if (gb.size() == 1) { if (!group_stride(gb[0], &m->b1_stride)) return false; }
    for (int64_t v : {m->off, m->m_stride, m->b0_stride, m->b1_stride})
      if ((v * ebytes) % 16 != 0) return false;
    for (auto& kv : st_) {
      bool known_sym = false;
      for (auto* d : {&dm, &dn}) for (auto& sy : d->syms) known_sym |= sy.first == kv.first;
      for (auto& d : gb) for (auto& sy : d.syms) known_sym |= sy.first == kv.first;
      if (!known_sym && kv.second != 0) return false;
    }
    m->elem_bytes = ebytes;
    return true;
  };
  std::vector<OutMap> in_maps;       // row operands of the epilogue that arrive by TMA (at most one)
  std::string tma_in_wait;           // code at the top of the epilogue step that takes the operand's chunk out of its tile

  // ---- operands of the epilogue that run along n (bias[n], mask[s, n], a residual x[b, s, n]):
  //      pre-loaded into a register tile with 16-byte loads, so that the per-column code has no
  //      dependent global load in it
  std::string load_code, tile_decls;
  int n_in_tiles = 0;
  std::set<int> not_loadable = {set.tn};
  auto collect_loads = [&](const Scalar& root, const std::map<std::string, std::string>* ren) {
    std::function<void(const Scalar&)> go = [&](const Scalar& e) {
      if (e.kind == Scalar::LocalScope) return;
      if (e.kind == Scalar::Get && !not_loadable.count(e.tn) && !n_sym.empty() && !e.idcs.empty()) {
        const Tnode& t = P.tn(e.tn);
        Indices canon = e.idcs;
        bool ok = t.mode != Mode::Virtual && (t.prec == Prec::Single || prec_bytes(t.prec) == 2) && t.prec != Prec::Uint16;
        for (auto& ix : canon) {
          if (ix.kind == Index::Iter) {
            if (ren) {
              auto it = ren->find(ix.sym);
              if (it != ren->end()) ix.sym = it->second;
            }
          } else if (ix.kind != Index::Fixed) ok = false;
        }
        Indices row;
        if (ok && along_n(canon, t.dims, &row)) {
          bool dup = false;
          for (auto& lt : em.load_tiles)
            if (lt.tn == e.tn && lt.idcs.size() == e.idcs.size()) {
              bool same = true;
              for (size_t a = 0; a < e.idcs.size(); ++a)
                if (lt.idcs[a].kind != e.idcs[a].kind || lt.idcs[a].sym != e.idcs[a].sym || lt.idcs[a].fixed != e.idcs[a].fixed) same = false;
              if (same) dup = true;
            }
          if (ok && !dup && n_in_tiles < 4) {
            const std::string member = "i" + std::to_string(n_in_tiles++);
            const std::string arr = "b200_t." + member;
            const std::string T = Emitter::ctype(t.prec);
            const bool f32 = t.prec == Prec::Single;
            std::ostringstream lc;
            // a 16-byte piece `q` (index v of the chunk's row) into the tile's entries
            std::string unpack;
            if (!pair && f32)
              unpack = "        " + arr + "[4 * v] = __uint_as_float(q.x); " + arr + "[4 * v + 1] = __uint_as_float(q.y);\n"
                       "        " + arr + "[4 * v + 2] = __uint_as_float(q.z); " + arr + "[4 * v + 3] = __uint_as_float(q.w);\n";
            else if (!pair)
              unpack = "        " + arr + "[8 * v] = (unsigned short)q.x; " + arr + "[8 * v + 1] = (unsigned short)(q.x >> 16);\n"
                       "        " + arr + "[8 * v + 2] = (unsigned short)q.y; " + arr + "[8 * v + 3] = (unsigned short)(q.y >> 16);\n"
                       "        " + arr + "[8 * v + 4] = (unsigned short)q.z; " + arr + "[8 * v + 5] = (unsigned short)(q.z >> 16);\n"
                       "        " + arr + "[8 * v + 6] = (unsigned short)q.w; " + arr + "[8 * v + 7] = (unsigned short)(q.w >> 16);\n";
            else if (f32)
              unpack = "        " + arr + "[2 * v] = b200_f2{__uint_as_float(q.x), __uint_as_float(q.y)};\n"
                       "        " + arr + "[2 * v + 1] = b200_f2{__uint_as_float(q.z), __uint_as_float(q.w)};\n";
            else
              unpack = "        " + arr + "[4 * v] = q.x; " + arr + "[4 * v + 1] = q.y; " + arr + "[4 * v + 2] = q.z; " + arr + "[4 * v + 3] = q.w;\n";
            const std::string V16 = f32 ? "4" : "8";   // elements per 16 bytes
            // An operand that varies with the row (a residual, a mask): per-thread row loads touch 32
            // lines per instruction.  When the node is a regular array for this contraction its chunk
            // (32 rows x the chunk's columns) arrives by one TMA load into a per-warp tile, a chunk
            // ahead like the register loads, and every lane takes its row out of the swizzled tile.
            OutMap imap;
            const bool by_tma = in_maps.empty() && make_map(e.tn, canon, &imap);   // (a stage that adds partial tiles never gets the TMA flag)
            if (by_tma) {
              in_maps.push_back(imap);
              lc << "  if (b200_es.tma) {\n    if ((threadIdx.x & 31u) == 0u) {\n"
                 << "      b200_mbar_expect_tx(b200_es.lbar, 32u * B200_EPI_CHUNK * " << prec_bytes(t.prec) << "u);\n"
                 << "      b200_tma_load_4d(b200_smem_addr(b200_es.ltile), b200_imap0, b200_es.lbar, (int)b200_n0, (int)(b200_m - (threadIdx.x & 31u)), (int)b200_b1, (int)b200_b0);\n"
                 << "    }\n  } else\n";
              tma_in_wait = "  if (b200_es.tma) {\n    b200_wait(b200_es.lbar, b200_es.lph, b200_es.abort_flag, b200_es.status, 5u);\n    b200_es.lph ^= 1u;\n"
                            "    constexpr int G = B200_EPI_CHUNK / " + V16 + ";\n#pragma unroll\n    for (int v = 0; v < G; ++v) {\n"
                            "        const uint4 q = b200_es.ltile[b200_lane * G + (v ^ B200_STAGE_KEY(b200_lane, G))];\n" + unpack +
                            "    }\n    __syncwarp();\n  }\n";
            }
            if (!pair) {
            tile_decls += std::string("  ") + T + " " + member + "[B200_EPI_CHUNK];\n";
            lc << "  if (b200_row_ok) {\n"
               << "    const " << T << "* b200_p = " << t.ident << " + (" << em.offset(row, t.dims) << ") + b200_n0;\n"
               << "    if (b200_n0 + B200_EPI_CHUNK <= b200_N && (((unsigned long long)b200_p) & 15ull) == 0ull) {\n"
               << "#pragma unroll\n      for (int v = 0; v < B200_EPI_CHUNK / " << V16 << "; ++v) {\n"
               << "        const uint4 q = ((const uint4*)b200_p)[v];\n" << unpack;
            lc << "      }\n    } else {\n#pragma unroll\n      for (int j = 0; j < B200_EPI_CHUNK; ++j) " << arr
               << "[j] = (b200_n0 + (unsigned int)j < b200_N) ? b200_p[j] : (" << T << ")0;\n    }\n  }\n";
            } else {
            // one pair per entry: packed words are taken as they lie in memory
            tile_decls += std::string("  ") + Emitter::pair_type(t.prec) + " " + member + "[B200_EPI_CHUNK / 2];\n";
            lc << "  if (b200_row_ok) {\n"
               << "    const " << T << "* b200_p = " << t.ident << " + (" << em.offset(row, t.dims) << ") + b200_n0;\n"
               << "    if (b200_n0 + B200_EPI_CHUNK <= b200_N && (((unsigned long long)b200_p) & 15ull) == 0ull) {\n"
               << "#pragma unroll\n      for (int v = 0; v < B200_EPI_CHUNK / " << V16 << "; ++v) {\n"
               << "        const uint4 q = ((const uint4*)b200_p)[v];\n" << unpack;
            lc << "      }\n    } else {\n#pragma unroll\n      for (int j = 0; j < B200_EPI_CHUNK / 2; ++j) {\n"
               << "        const " << T << " b200_e0 = (b200_n0 + 2u * (unsigned int)j < b200_N) ? b200_p[2 * j] : (" << T << ")0;\n"
               << "        const " << T << " b200_e1 = (b200_n0 + 2u * (unsigned int)j + 1u < b200_N) ? b200_p[2 * j + 1] : (" << T << ")0;\n";
            if (f32) lc << "        " << arr << "[j] = b200_f2{b200_e0, b200_e1};\n";
            else lc << "        " << arr << "[j] = (unsigned int)b200_e0 | ((unsigned int)b200_e1 << 16);\n";
            lc << "      }\n    }\n  }\n";
            }
            load_code += lc.str();
            em.load_tiles.push_back({e.tn, e.idcs, arr + "[b200_j]"});
            em.used_nodes.insert(e.tn);
          }
        }
      }
      if (e.kind == Scalar::GetDyn) return;
      for (auto& a : e.args) go(*a.s);
    };
    go(root);
  };
  if (!form_b) collect_loads(*set.value, nullptr);

  em.scope_subst[kAccScope] = "b200_acc";
  if (pair && !form_b) {
    em.scope_subst[scope->scope_id] = "b200_acc";
    if (!em.pair_supported(*set.value)) return false;
  }
  std::string body;
  add_out(set.tn, set.idcs);
  if (form_b && opt.enable_splitk && outs[0].unit_n) {
    g.may_split = true;
    g.split_k = gemm_split_k(g);
  }
  const bool reds = g.split_k > 1;   // partial tiles are added to the output instead of stored
  if (form_b) {
    const Tnode& t = D;
    std::string off = em.offset(set.idcs, t.dims);
    if (reds) body = "      " + outs[0].arr + "[b200_j] = b200_acc;\n";
    else if (g.accumulate) body = "      " + outs[0].arr + "[b200_j] = " + t.ident + "[" + off + "] + b200_acc;\n";
    else body = "      " + outs[0].arr + "[b200_j] = b200_acc;\n";
  } else {
    em.scope_subst[scope->scope_id] = "b200_acc";
    body = em.stmt(set, 6);
  }
  em.forwarded[set.tn] = {set.idcs, outs[0].arr + "[b200_j]"};

  // ---- fuse following pointwise assignments over the same index space into the epilogue:
  //      `for f'.. { u[f'..] := E(t[f'..], ...) }` where t is what this stage just produced
  int fused = 0;
  std::string aliases;
  std::set<int> produced = {set.tn};
  for (const Follower& fo : followers) {
    if (reds) break;   // partial tiles cannot feed a follow-up assignment
    if (fo.nest.size() != free_loops.size() || fo.set->kind != Stmt::Set || fo.set->vec_len > 0) break;
    bool ok = true;
    std::map<std::string, std::string> ren;  // follower symbol -> this stage's symbol
    for (size_t i = 0; i < fo.nest.size(); ++i) {
      if (fo.nest[i].from != 0 || fo.nest[i].extent() != free_loops[i].extent()) ok = false;
      ren[fo.nest[i].sym] = free_loops[i].sym;
    }
    if (!ok) break;
    auto renamed_equal = [&](const Indices& a, const Indices& b) {
      if (a.size() != b.size()) return false;
      for (size_t i = 0; i < a.size(); ++i) {
        if (a[i].kind != b[i].kind) return false;
        if (a[i].kind == Index::Iter) {
          auto it = ren.find(a[i].sym);
          if ((it == ren.end() ? a[i].sym : it->second) != b[i].sym) return false;
        } else if (a[i].kind == Index::Fixed) {
          if (a[i].fixed != b[i].fixed) return false;
        } else return false;
      }
      return true;
    };
    // the follower may read produced nodes only at the very position being produced, writes a
    // node not produced or read so far, at a position that is a bijection of the index space
    bool reads_producer = false;
    std::function<void(const Scalar&)> chk = [&](const Scalar& e) {
      if (e.kind == Scalar::LocalScope || e.kind == Scalar::GetLocal || e.kind == Scalar::GetMerge) ok = false;
      if (e.kind == Scalar::Get || e.kind == Scalar::GetDyn) {
        if (produced.count(e.tn)) {
          reads_producer = true;
          const Out* src = nullptr;
          for (auto& o : outs)
            if (o.tn == e.tn) src = &o;
          if (e.kind != Scalar::Get || !src || !renamed_equal(e.idcs, src->idcs)) ok = false;
        }
        if (e.tn == fo.set->tn) ok = false;
      }
      for (auto& a : e.args) chk(*a.s);
    };
    chk(*fo.set->value);
    if (!ok || !reads_producer || produced.count(fo.set->tn) || em.used_nodes.count(fo.set->tn)) break;
    if (pair && !em.pair_supported(*fo.set->value)) return false;   // the one-column form can still fuse it
    for (size_t i = 0; i < fo.nest.size(); ++i) {
      int occ = 0;
      for (auto& ix : fo.set->idcs)
        if (ix.kind == Index::Iter && ix.sym == fo.nest[i].sym) ++occ;
      if (occ != 1) ok = false;
    }
    for (auto& ix : fo.set->idcs)
      if (ix.kind != Index::Iter && ix.kind != Index::Fixed) ok = false;
    if (!ok) break;
    // aliases make the follower's symbols names for this stage's symbols
    for (size_t i = 0; i < fo.nest.size(); ++i)
      if (fo.nest[i].sym != free_loops[i].sym)
        aliases += "      const unsigned int " + fo.nest[i].sym + " = " + free_loops[i].sym + ";\n";
    // forwarded reads are matched on the follower's own spelling of the indices
    for (auto& o : outs) {
      Indices spelled = o.idcs;
      for (auto& ix : spelled)
        if (ix.kind == Index::Iter)
          for (auto& kv : ren)
            if (kv.second == ix.sym) ix.sym = kv.first;
      em.forwarded[o.tn] = {spelled, o.arr + "[b200_j]"};
    }
    Indices canon = fo.set->idcs;
    for (auto& ix : canon)
      if (ix.kind == Index::Iter) ix.sym = ren[ix.sym];
    add_out(fo.set->tn, canon);
    em.set_redirect[fo.set->tn] = {fo.set->idcs, outs.back().arr + "[b200_j]"};
    not_loadable.insert(fo.set->tn);
    for (auto& o : outs) not_loadable.insert(o.tn);
    collect_loads(*fo.set->value, &ren);
    body += aliases + em.stmt(*fo.set, 6);
    aliases.clear();
    produced.insert(fo.set->tn);
    ++fused;
  }
  // ---- row followers.  When the whole output row fits one epilogue chunk (N <= 32: the logits of
  //      a classifier), the thread that owns accumulator row m holds that row of every produced
  //      node in registers, so assignments over whole rows can run right there: a row maximum,
  //      `exp(x - max)`, a row sum (the softmax pieces of lib/nn_blocks.ml:137-143), each a loop
  //      nest over the row loops with an optional trailing loop over the N columns, reading the
  //      produced rows and anything else from memory.  A last assignment may sum over ALL rows and
  //      columns (the mean cross-entropy): every epilogue warp leaves the partial sum of its 32
  //      rows in scratch, the warp that takes the last ticket adds the partials in slot order -- a
  //      fixed order, so the value does not depend on scheduling -- and evaluates the assignment.
  struct RowNode {
    int tn;
    Indices canon;      // indices in this stage's symbols
    int n_axis;         // axis carrying the n symbol, -1 for one value per row
    std::string name;   // register array / scalar
    bool from_main;     // the main output's tile (already stored by the column loop's store path)
  };
  std::vector<RowNode> rownodes;
  std::string row_code, row_decls, row_stores, final_code;
  std::set<int> row_written;   // nodes the row followers write
  int row_fused = 0;
  size_t scratch_bytes = 0;
  const int64_t N = g.n.extent;
  {
    std::vector<LoopDim> row_loops;
    for (auto& d : free_loops) {
      bool is_n = false;
      for (auto& sy : dn.syms) is_n = is_n || sy.first == d.sym;
      if (!is_n) row_loops.push_back(d);
    }
    int bn_t;
    bool pair_t;
    gemm_tile_shape(g, &bn_t, &pair_t);
    bool can = !pair && !reds && !(form_b && g.accumulate) && n_syms == 1 && N <= 32 && bn_t <= 32 && !pair_t && outs[0].unit_n;
    if (can) {
      int na = -1;
      for (size_t a = 0; a < set.idcs.size(); ++a)
        if (set.idcs[a].kind == Index::Iter && set.idcs[a].sym == n_sym) na = (int)a;
      rownodes.push_back({set.tn, set.idcs, na, outs[0].arr, true});
      can = na >= 0;
    }
    std::set<int> row_produced;
    for (auto& o : outs) row_produced.insert(o.tn);
    for (size_t fi = (size_t)fused; can && fi < followers.size(); ++fi) {
      if (outs.size() != 1) break;   // only directly after the contraction's own assignment
      const Follower& fo = followers[fi];
      if (!fo.set || fo.set->kind != Stmt::Set || fo.set->vec_len > 0) break;
      const bool global = fo.nest.empty();
      std::map<std::string, std::string> ren;     // follower symbol -> this stage's symbol
      std::set<std::string> col_syms;             // follower symbols that run over the N columns
      std::string col_loop;                       // the follower's own trailing column loop, if any
      bool ok = true;
      if (!global) {
        if (fo.nest.size() != row_loops.size() && fo.nest.size() != row_loops.size() + 1) break;
        for (size_t i = 0; i < row_loops.size(); ++i) {
          if (fo.nest[i].from != 0 || fo.nest[i].extent() != row_loops[i].extent()) ok = false;
          ren[fo.nest[i].sym] = row_loops[i].sym;
        }
        if (fo.nest.size() == row_loops.size() + 1) {
          const LoopDim& c = fo.nest.back();
          if (c.from != 0 || c.extent() != N) ok = false;
          col_loop = c.sym;
          col_syms.insert(c.sym);
        }
      }
      if (!ok) break;
      // local scopes: `[v := neutral;] for c' < N { v := v op term }`; the global form sums over
      // (row loops, c')
      const Scalar* gscope = nullptr;
      std::vector<const Scalar*> scopes;
      std::function<void(const Scalar&)> find_scopes = [&](const Scalar& e) {
        if (e.kind == Scalar::LocalScope) { scopes.push_back(&e); return; }
        for (auto& a : e.args) find_scopes(*a.s);
      };
      find_scopes(*fo.set->value);
      if (global && scopes.size() != 1) break;
      std::vector<LoopDim> gloops;
      const Stmt* gstep = nullptr;
      for (auto* sc : scopes) {
        const Stmt* b = sc->body.get();
        if (b->kind == Stmt::Seq) {
          if (b->items.size() != 2 || b->items[0]->kind != Stmt::SetLocal || b->items[0]->value->kind != Scalar::Const) { ok = false; break; }
          b = b->items[1].get();
        }
        std::vector<LoopDim> red;
        while (b->kind == Stmt::For) { red.push_back({b->index, b->from, b->to}); b = b->body.get(); }
        if (b->kind != Stmt::SetLocal || b->scope_id != sc->scope_id) { ok = false; break; }
        bool nested = false;
        walk_scalar_simple(*b->value, [&](const Scalar& x) { if (x.kind == Scalar::LocalScope) nested = true; });
        if (nested) { ok = false; break; }
        if (global) {
          if (red.size() != row_loops.size() + 1) { ok = false; break; }
          for (size_t i = 0; i < row_loops.size(); ++i) {
            if (red[i].from != 0 || red[i].extent() != row_loops[i].extent()) ok = false;
            ren[red[i].sym] = row_loops[i].sym;
          }
          if (red.back().from != 0 || red.back().extent() != N) ok = false;
          col_syms.insert(red.back().sym);
          // the step must be a plain sum: v := v + term / term + v / fma(a, b, v), from zero
          const Scalar& v = *b->value;
          auto is_self = [&](const Scalar& e) { return e.kind == Scalar::GetLocal && e.scope_id == sc->scope_id; };
          bool sum = (v.kind == Scalar::Bin && v.op == "add" && (is_self(*v.args[0].s) != is_self(*v.args[1].s))) ||
                     (v.kind == Scalar::Tern && v.op == "fma" && is_self(*v.args[2].s));
          const Stmt* sb = sc->body.get();
          if (sb->kind == Stmt::Seq && sb->items[0]->value->cval != 0.0) sum = false;
          if (!sum || P.tn(sc->tn).prec != Prec::Single) ok = false;
          gscope = sc;
          gloops = red;
          gstep = b;
        } else {
          if (red.size() != 1 || red[0].from != 0 || red[0].extent() != N) { ok = false; break; }
          col_syms.insert(red[0].sym);
        }
      }
      if (!ok) break;
      // reads: produced nodes only row-locally; no merge buffer; a read of the written node is out
      auto chk = [&](const Scalar& e) {
        if (e.kind == Scalar::GetMerge) ok = false;
        if (e.kind == Scalar::Get || e.kind == Scalar::GetDyn) {
          if (e.tn == fo.set->tn) ok = false;
          if (row_produced.count(e.tn)) {
            const RowNode* rn = nullptr;
            for (auto& r : rownodes) if (r.tn == e.tn) rn = &r;
            if (e.kind != Scalar::Get || !rn || e.idcs.size() != rn->canon.size()) { ok = false; return; }
            for (size_t a = 0; a < e.idcs.size(); ++a) {
              Index x = e.idcs[a];
              if ((int)a == rn->n_axis) {
                if (!(x.kind == Index::Fixed && x.fixed >= 0 && x.fixed < N) && !(x.kind == Index::Iter && col_syms.count(x.sym))) ok = false;
              } else {
                if (x.kind == Index::Iter && ren.count(x.sym)) x.sym = ren[x.sym];
                const Index& y = rn->canon[a];
                if (x.kind != y.kind || x.sym != y.sym || x.fixed != y.fixed || x.terms != y.terms) ok = false;
              }
            }
          }
        }
      };
      walk_scalar_simple(*fo.set->value, chk);
      if (!ok || row_produced.count(fo.set->tn) || em.used_nodes.count(fo.set->tn)) break;
      const Tnode& T = P.tn(fo.set->tn);
      if (T.mode == Mode::Virtual || T.prec == Prec::Uint4x32) break;
      if (global) {
        // written position: fixed indices only
        for (auto& ix : fo.set->idcs) if (ix.kind != Index::Fixed) ok = false;
        if (!ok) break;
        em.row_ren = ren;
        em.row_forwards.clear();
        for (auto& r : rownodes) em.row_forwards.push_back({r.tn, r.canon, r.n_axis, r.name, ""});
        em.unroll_loops = true;
        std::string code = "  {\n    float b200_part = 0.0f;\n    if (b200_row_ok) {\n";
        for (size_t i = 0; i < row_loops.size(); ++i)
          if (gloops[i].sym != row_loops[i].sym)
            code += "      const unsigned int " + gloops[i].sym + " = " + row_loops[i].sym + ";\n";
        em.scope_subst[gscope->scope_id] = "b200_part";
        code += "#pragma unroll\n      for (unsigned int " + gloops.back().sym + " = 0; " + gloops.back().sym + " < " + std::to_string(N) + "u; ++" +
                gloops.back().sym + ") {\n" + em.stmt(*gstep, 8) + "      }\n    }\n";
        // per-warp partial, ticket, ordered combine by the last warp
        code += "    b200_part = b200_warp_sum(b200_part);\n"
                "    float* b200_slots = (float*)b200_partials;\n"
                "    unsigned int* b200_ticket = (unsigned int*)(b200_partials + 4ull * b200_nslots);\n"
                "    unsigned int b200_last = 0u;\n"
                "    if (b200_lane == 0u) {\n      b200_slots[b200_slot] = b200_part;\n      __threadfence();\n"
                "      b200_last = atomicAdd(b200_ticket, 1u) == b200_nslots - 1u ? 1u : 0u;\n    }\n"
                "    b200_last = __shfl_sync(0xffffffffu, b200_last, 0);\n"
                "    if (b200_last) {\n      __threadfence();\n      float b200_total = 0.0f;\n"
                "      for (unsigned int b200_i = b200_lane; b200_i < b200_nslots; b200_i += 32u) b200_total += ((volatile float*)b200_slots)[b200_i];\n"
                "      b200_total = b200_warp_sum(b200_total);\n      if (b200_lane == 0u) {\n";
        em.scope_subst[gscope->scope_id] = "b200_total";
        Emitter::Res v = em.scalar(T.prec, *fo.set->value);
        if (!v.defs.empty()) { em.scope_subst.erase(gscope->scope_id); break; }
        em.used_nodes.insert(fo.set->tn);
        row_written.insert(fo.set->tn);
        const std::string gv = "b200_g" + std::to_string(fo.set->tn);
        code += "        const " + std::string(Emitter::rtype(T.prec)) + " " + gv + " = " + v.expr + ";\n"
                "        " + T.ident + "[" + em.offset(fo.set->idcs, T.dims) + "] = " + Emitter::store_wrap(T.prec, gv) + ";\n";
        em.scope_subst.erase(gscope->scope_id);
        // Scalar assignments that follow the sum (a mean: total / batch) run right here, in the one
        // thread that holds the total: they read it (and one another) from registers and otherwise
        // only nodes this stage does not write.
        {
          const auto saved_fwd = em.forwarded;
          em.forwarded[fo.set->tn] = {fo.set->idcs, gv};
          std::set<int> stage_writes = row_written;
          for (auto& o : outs) stage_writes.insert(o.tn);
          stage_writes.insert(fo.set->tn);
          for (size_t fj = fi + 1; fj < followers.size(); ++fj) {
            const Follower& ft = followers[fj];
            if (!ft.set || ft.set->kind != Stmt::Set || ft.set->vec_len > 0 || !ft.nest.empty()) break;
            const Tnode& T2 = P.tn(ft.set->tn);
            if (T2.mode == Mode::Virtual || T2.prec == Prec::Uint4x32 || stage_writes.count(ft.set->tn) || em.used_nodes.count(ft.set->tn)) break;
            bool fine = true;
            for (auto& ix : ft.set->idcs) if (ix.kind != Index::Fixed) fine = false;
            walk_scalar_simple(*ft.set->value, [&](const Scalar& e) {
              if (e.kind == Scalar::LocalScope || e.kind == Scalar::GetLocal || e.kind == Scalar::GetMerge || e.kind == Scalar::GetDyn) fine = false;
              if (e.kind == Scalar::Get) {
                for (auto& ix : e.idcs) if (ix.kind != Index::Fixed) fine = false;
                auto fw = em.forwarded.find(e.tn);
                const bool forwarded_here = fw != em.forwarded.end() && fw->second.first.size() == e.idcs.size() &&
                                            std::equal(e.idcs.begin(), e.idcs.end(), fw->second.first.begin(),
                                                       [](const Index& a, const Index& b) { return a.kind == b.kind && a.fixed == b.fixed; });
                if (stage_writes.count(e.tn) && !forwarded_here) fine = false;   // another CTA may still be writing it
              }
            });
            if (!fine) break;
            Emitter::Res w = em.scalar(T2.prec, *ft.set->value);
            if (!w.defs.empty()) break;
            const std::string tv = "b200_g" + std::to_string(ft.set->tn);
            code += "        const " + std::string(Emitter::rtype(T2.prec)) + " " + tv + " = " + w.expr + ";\n"
                    "        " + T2.ident + "[" + em.offset(ft.set->idcs, T2.dims) + "] = " + Emitter::store_wrap(T2.prec, tv) + ";\n";
            em.used_nodes.insert(ft.set->tn);
            row_written.insert(ft.set->tn);
            stage_writes.insert(ft.set->tn);
            em.forwarded[ft.set->tn] = {ft.set->idcs, tv};
            ++row_fused;
          }
          em.forwarded = saved_fwd;
        }
        code += "        *b200_ticket = 0u;\n      }\n    }\n  }\n";
        em.unroll_loops = false;
        final_code = code;
        // slots: one per epilogue warp of every tile (4 warps per 128-row tile)
        long long tiles = (g.m.extent + 127) / 128;
        for (auto& b : g.batch) tiles *= b.extent;
        scratch_bytes = (size_t)tiles * 4 * 4 + 16;
        ++row_fused;
        break;   // the global sum ends the epilogue
      }
      // written position: every row symbol once, the column loop at most once, fixed otherwise
      Indices canon = fo.set->idcs;
      int na = -1;
      {
        std::map<std::string, int> seen;
        for (size_t a = 0; a < canon.size(); ++a) {
          Index& ix = canon[a];
          if (ix.kind == Index::Fixed) continue;
          if (ix.kind != Index::Iter) { ok = false; break; }
          if (!col_loop.empty() && ix.sym == col_loop) { if (na >= 0) ok = false; na = (int)a; ix.sym = n_sym; continue; }
          auto it = ren.find(ix.sym);
          if (it == ren.end()) { ok = false; break; }
          ix.sym = it->second;
          if (++seen[ix.sym] > 1) ok = false;
        }
        for (auto& d : row_loops) if (d.extent() > 1 && !seen.count(d.sym)) ok = false;
        if (!col_loop.empty() && na < 0) ok = false;
      }
      if (!ok) break;
      const std::string name = "b200_f" + std::to_string(fo.set->tn);
      em.row_ren = ren;
      em.row_forwards.clear();
      for (auto& r : rownodes) em.row_forwards.push_back({r.tn, r.canon, r.n_axis, r.name, ""});
      em.unroll_loops = true;
      const auto saved_redirect = em.set_redirect;
      em.set_redirect[fo.set->tn] = {fo.set->idcs, na >= 0 ? name + "[" + col_loop + "]" : name};
      std::string code = "    {\n";
      for (size_t i = 0; i < row_loops.size(); ++i)
        if (fo.nest[i].sym != row_loops[i].sym)
          code += "      const unsigned int " + fo.nest[i].sym + " = " + row_loops[i].sym + ";\n";
      std::string st_text = em.stmt(*fo.set, 8);
      if (na >= 0)
        code += "#pragma unroll\n      for (unsigned int " + col_loop + " = 0; " + col_loop + " < " + std::to_string(N) + "u; ++" + col_loop +
                ") {\n" + st_text + "      }\n";
      else
        code += st_text;
      code += "    }\n";
      em.set_redirect = saved_redirect;
      em.unroll_loops = false;
      em.used_nodes.insert(fo.set->tn);
      row_decls += std::string("  ") + Emitter::rtype(T.prec) + " " + name + (na >= 0 ? "[" + std::to_string(N) + "]" : std::string()) + ";\n";
      row_code += code;
      // the node's store: a thread writes its own row
      {
        Indices at = canon;
        if (na >= 0) { at[(size_t)na].kind = Index::Fixed; at[(size_t)na].fixed = 0; at[(size_t)na].sym.clear(); }
        const std::string off = em.offset(at, T.dims);
        if (na >= 0) {
          int64_t stride = 1;
          for (size_t a = (size_t)na + 1; a < T.dims.size(); ++a) stride *= T.dims[a];
          row_stores += "#pragma unroll\n    for (unsigned int b200_c = 0; b200_c < " + std::to_string(N) + "u; ++b200_c) " + T.ident + "[(" + off +
                        ") + b200_c * " + std::to_string(stride) + "u] = " + Emitter::store_wrap(T.prec, name + "[b200_c]") + ";\n";
        } else {
          row_stores += "    " + T.ident + "[" + off + "] = " + Emitter::store_wrap(T.prec, name) + ";\n";
        }
      }
      rownodes.push_back({fo.set->tn, canon, na, name, false});
      row_produced.insert(fo.set->tn);
      row_written.insert(fo.set->tn);
      ++row_fused;
    }
    em.row_forwards.clear();
    em.row_ren.clear();
  }
  fused += row_fused;
  *n_fused = fused;
  if (pair_fail) return false;

  // ---- outputs as TMA stores.  A chunk (32 rows of the warp x the chunk's columns) that sits in the
  // staging tile leaves with one copy instruction when the node is a regular [batch.., m, n] array
  // for this contraction: the m symbols (and each batch group's) compose to one stride, everything is
  // 16-byte aligned.  All of the stage's row-contiguous outputs must qualify (the staging tiles are
  // then managed for the copy engine), and partial tiles that are added to the output do not.
  std::vector<OutMap> out_maps;
  if (g.split_k == 1 && !(form_b && g.accumulate)) {
    bool all = true;
    std::vector<OutMap> maps;
    for (auto& o : outs) {
      const int ebytes = prec_bytes(P.tn(o.tn).prec);
      if (!(o.unit_n && (ebytes == 4 || ebytes == 2))) continue;   // stored element by element, no staging tile
      OutMap m;
      if (!make_map(o.tn, o.idcs, &m)) { all = false; break; }
      o.tma = (int)maps.size();
      maps.push_back(m);
    }
    if (all) out_maps = maps;
    else for (auto& o : outs) o.tma = -1;
  }

  std::ostringstream fn;
  // parameters of the epilogue: the nodes it touches (+ static table)
  std::string params, args;
  std::vector<KArg> kargs;
  for (auto& t : P.tnodes) {
    if (!em.used_nodes.count(t.id) || t.mode == Mode::Virtual) continue;
    bool written = false;
    for (auto& o : outs) written |= o.tn == t.id;
    written |= row_written.count(t.id) > 0;
    params += std::string(", ") + (written ? "" : "const ") + Emitter::ctype(t.prec) + "* " + (written ? "" : "__restrict__ ") + t.ident;
    args += ", " + t.ident;
    kargs.push_back({KArg::Node, t.id});
  }
  std::string statics_prologue;
  {
    std::string text = body + load_code + row_code + final_code;
    for (size_t i = 0; i < P.statics.size(); ++i) {
      const std::string& s = P.statics[i].sym;
      size_t p = 0;
      bool found = false;
      auto isid = [](char c) { return isalnum((unsigned char)c) || c == '_'; };
      while ((p = text.find(s, p)) != std::string::npos) {
        bool l = p == 0 || !isid(text[p - 1]);
        bool r = p + s.size() >= text.size() || !isid(text[p + s.size()]);
        if (l && r) { found = true; break; }
        p += s.size();
      }
      if (found) statics_prologue += "  const unsigned int " + s + " = b200_statics[" + std::to_string(i) + "];\n";
    }
    if (!statics_prologue.empty()) {
      params += ", const unsigned int* __restrict__ b200_statics";
      args += ", b200_statics";
      kargs.push_back({KArg::Statics, -1});
    }
  }
  if (scratch_bytes) {
    params += ", unsigned char* b200_partials";
    args += ", b200_partials";
    kargs.push_back({KArg::Scratch, 0});   // the planner assigns the offset into the routine's reduction scratch
  }
  if (em.uses_merge) return false;
  // tensor maps of the outputs: kernel parameters by value, pointers everywhere else
  std::string params_k = params, map_prologue;
  if (!in_maps.empty()) {
    params_k += ", const __grid_constant__ b200_tmap b200_imap0_k";
    params += ", const b200_tmap* b200_imap0";
    args += ", b200_imap0";
    map_prologue += "    const b200_tmap* b200_imap0 = &b200_imap0_k;\n";
    map_prologue += "    if (ew == 3u && lane == 0) asm volatile(\"prefetch.tensormap [%0];\" ::\"l\"((unsigned long long)b200_imap0) : \"memory\");\n";
  }
  for (size_t k = 0; k < out_maps.size(); ++k) {
    const std::string nm = "b200_omap" + std::to_string(k);
    params_k += ", const __grid_constant__ b200_tmap " + nm + "_k";
    params += ", const b200_tmap* " + nm;
    args += ", " + nm;
    map_prologue += "    const b200_tmap* " + nm + " = &" + nm + "_k;\n";
    map_prologue += "    if (ew == " + std::to_string(k % 4) + "u && lane == 0) asm volatile(\"prefetch.tensormap [%0];\" ::\"l\"((unsigned long long)" + nm + ") : \"memory\");\n";
  }

  std::string ptr_code;
  for (auto& o : outs) {
    const Tnode& t = P.tn(o.tn);
    const int ebytes = prec_bytes(t.prec);
    if (!(o.unit_n && (ebytes == 4 || ebytes == 2))) continue;
    const std::string G = std::string("(B200_EPI_CHUNK / ") + (ebytes == 4 ? "4" : "8") + ")";
    const std::string member = "r" + std::to_string(o.tn);
    tile_decls += "  unsigned long long " + member + "[" + G + "];\n";
    ptr_code += "  {\n"
                "    const unsigned long long b200_pv = b200_row_ok ? (unsigned long long)(" + t.ident + " + (" + o.row_off +
                ")) : 0ull;\n#pragma unroll\n    for (int it = 0; it < " + G + "; ++it) b200_t." + member +
                "[it] = __shfl_sync(0xffffffffu, b200_pv, it * (32 / " + G + ") + b200_lane / " + G + ");\n  }\n";
  }
  {
    // Operand tiles of one chunk.  They do not depend on the accumulator, so the kernel fills them
    // for a tile's first chunk while the tensor cores still work on it, and the epilogue refills
    // them for the next chunk as soon as it has consumed the current one (the loads then overlap
    // the stores).  Parameters mirror the epilogue's so that one argument list serves both.
    fn << "struct b200_in_tiles {\n" << tile_decls << (tile_decls.empty() ? "  int none;\n" : "") << "};\n"
       << "__device__ __forceinline__ void b200_epilogue_load(b200_in_tiles& b200_t, unsigned int b200_b0, unsigned int b200_b1, "
          "unsigned int b200_m, bool b200_row_ok, unsigned int b200_n0, unsigned int b200_N, b200_epi_state& b200_es"
       << params << ") {\n";
    if (!load_code.empty()) {
      fn << statics_prologue;
      ep.str("");
      if (gb.size() == 2) { recover(gb[0], "b200_b0"); recover(gb[1], "b200_b1"); }
      else if (gb.size() == 1) { recover(gb[0], "b200_b1"); }
      recover(dm, "b200_m");
      fn << ep.str() << unit_syms << load_code;
      ep.str("");
    }
    fn << "}\n";
    // Row pointers of the transposed store, once per tile: entry `it` is the address of column 0
    // of the row this lane writes in store step `it` (0 for rows beyond M).
    fn << "__device__ __forceinline__ void b200_epilogue_rows(b200_in_tiles& b200_t, unsigned int b200_b0, unsigned int b200_b1, "
          "unsigned int b200_m, bool b200_row_ok" << params << ") {\n";
    if (!ptr_code.empty()) {
      fn << statics_prologue << "  const unsigned int b200_lane = threadIdx.x & 31u;\n";
      ep.str("");
      if (gb.size() == 2) { recover(gb[0], "b200_b0"); recover(gb[1], "b200_b1"); }
      else if (gb.size() == 1) { recover(gb[0], "b200_b1"); }
      recover(dm, "b200_m");
      fn << ep.str() << unit_syms << ptr_code;
      ep.str("");
    }
    fn << "}\n";
  }
  // Staging swizzle.  A row of the staging tile holds G 16-byte groups, so 8 / G rows share one
  // 128-byte line of banks; the group index is xor-ed with a key that changes every 8 / G rows,
  // which makes the 8 lanes of a quarter warp (one row group each when writing, 8 / G rows of G
  // groups when reading) hit 8 different bank groups.
  fn << "__device__ __forceinline__ void b200_red_add_v4(unsigned long long addr, uint4 q) {\n"
        "  asm volatile(\"red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\" ::\"l\"(addr), \"f\"(__uint_as_float(q.x)), \"f\"(__uint_as_float(q.y)),\n"
        "               \"f\"(__uint_as_float(q.z)), \"f\"(__uint_as_float(q.w)) : \"memory\");\n}\n";
  fn << "#define B200_STAGE_KEY(row, G) ((G) >= 8 ? ((row) & 7u) : (((row) / (8u / ((G) >= 8 ? 8u : (G)))) % (G)))\n";
  // developer trace: the first epilogue thread of CTA 0 adds up the clock cycles it spends in
  // each phase of the epilogue (slot = phase that just ended)
  fn << "#ifdef B200_TRACE\n__device__ __forceinline__ void b200_tre(int slot, bool dump, unsigned int* out) {\n"
        "  __shared__ unsigned int acc[16];\n  __shared__ long long last;\n"
        "  if (blockIdx.x != 0 || threadIdx.x != 64) return;\n"
        "  if (dump) { for (int i = 0; i < 16; ++i) { out[16 + i] = acc[i]; } return; }\n"
        "  const long long now = clock64();\n"
        "  if (slot < 0) { for (int i = 0; i < 16; ++i) acc[i] = 0; } else { acc[slot] += (unsigned int)(now - last); }\n"
        "  last = clock64();\n}\n"
        "#define B200_TRE(slot) b200_tre(slot, false, nullptr)\n"
        "#else\n#define B200_TRE(slot) do { } while (0)\n#endif\n"
     << "__device__ __forceinline__ void b200_tmem_ld_chunk(unsigned int taddr, unsigned int* r);\n"
     << "__device__ __forceinline__ void b200_epilogue_row(unsigned int* b200_r, unsigned int b200_b0, unsigned int b200_b1, "
        "unsigned int b200_m, bool b200_row_ok, unsigned int b200_n0, unsigned int b200_N, uint4* b200_stage, "
        "bool b200_has_next, unsigned int b200_next_taddr, b200_in_tiles& b200_t, unsigned int b200_slot, unsigned int b200_nslots, "
        "bool b200_nx_ok, unsigned int b200_nx_b0, unsigned int b200_nx_b1, unsigned int b200_nx_m, bool b200_nx_row_ok, unsigned int b200_nx_n0, "
        "b200_epi_state& b200_es"
     << params << ") {\n"
     << statics_prologue;
  fn << "  const unsigned int b200_lane = threadIdx.x & 31u;\n" << tma_in_wait;
  {
    // batch axes: gb[0] is the outer one
    ep.str("");
    if (gb.size() == 2) { recover(gb[0], "b200_b0"); recover(gb[1], "b200_b1"); }
    else if (gb.size() == 1) { recover(gb[0], "b200_b1"); }
    recover(dm, "b200_m");
    fn << ep.str();
    ep.str("");
  }
  fn << unit_syms;
  // output tiles hold expression values (16-bit precisions as rounded floats); they are packed at the store
  // The arithmetic of rows beyond M and columns beyond N is skipped only when it reads memory
  // itself; when every operand comes from a register tile it runs on whatever the registers hold
  // (nothing of it is stored), which saves a possibly divergent branch per column.
  const std::string guard = (em.direct_reads > 0 || (form_b && g.accumulate && g.split_k == 1)) ? "b200_row_ok && b200_n < b200_N" : "true";
  if (pair) {
    for (auto& o : outs) fn << "  " << Emitter::pair_type(P.tn(o.tn).prec) << " " << o.arr << "[B200_EPI_CHUNK / 2];\n";
    fn << "#pragma unroll\n  for (int b200_j = 0; b200_j < B200_EPI_CHUNK / 2; ++b200_j) {\n"
       << "    const unsigned int b200_n = b200_n0 + 2u * (unsigned int)b200_j;\n"
       << "    if (" << guard << ") {\n"
       << "      const b200_f2 b200_acc = {__uint_as_float(b200_r[2 * b200_j]), __uint_as_float(b200_r[2 * b200_j + 1])};\n";
  } else {
  for (auto& o : outs) fn << "  " << Emitter::rtype(P.tn(o.tn).prec) << " " << o.arr << "[B200_EPI_CHUNK];\n";
  fn << "#pragma unroll\n  for (int b200_j = 0; b200_j < B200_EPI_CHUNK; ++b200_j) {\n"
     << "    const unsigned int b200_n = b200_n0 + (unsigned int)b200_j;\n"
     << "    if (" << guard << ") {\n"
     << "      const float b200_acc = __uint_as_float(b200_r[b200_j]);\n";
  }
  recover(dn, "b200_n");
  fn << ep.str() << body << "    }\n  }\n";
  // the accumulator chunk is consumed: start fetching the next one while this one is stored
  // ... or, after the tile's last chunk, the operand tiles of the first chunk of this warp's NEXT
  // tile: their latency then hides behind this chunk's stores and the wait for the next accumulator
  fn << "  B200_TRE(13);\n  if (b200_has_next) {\n    b200_tmem_ld_chunk(b200_next_taddr, b200_r);\n"
     << "    b200_epilogue_load(b200_t, b200_b0, b200_b1, b200_m, b200_row_ok, b200_n0 + B200_EPI_CHUNK, b200_N, b200_es" << args << ");\n"
     << "  } else if (b200_nx_ok) {\n"
     << "    b200_epilogue_load(b200_t, b200_nx_b0, b200_nx_b1, b200_nx_m, b200_nx_row_ok, b200_nx_n0, b200_N, b200_es" << args << ");\n  }\n  B200_TRE(10);\n";
  // ---- store the register tiles.  A thread owns one row of the chunk, so storing from
  //      registers would touch 32 different lines per instruction; when the chunk is whole,
  //      contiguous and every row is 16-byte aligned, the warp transposes the chunk through a
  //      swizzled shared-memory staging tile and writes whole row segments instead.
  // the chunk of one output into the staging tile `b200_tile` (G 16-byte groups per row)
  auto sts_code = [&](const Out& o) {
    const Tnode& t = P.tn(o.tn);
    const int ebytes = prec_bytes(t.prec);
    std::ostringstream fn;
    fn << "#pragma unroll\n      for (int g = 0; g < G; ++g) {\n        uint4 q;\n";
    if (pair && ebytes == 4) {
      fn << "        q.x = __float_as_uint(" << o.arr << "[2 * g].x); q.y = __float_as_uint(" << o.arr << "[2 * g].y);\n"
         << "        q.z = __float_as_uint(" << o.arr << "[2 * g + 1].x); q.w = __float_as_uint(" << o.arr << "[2 * g + 1].y);\n";
    } else if (pair) {
      fn << "        q.x = " << o.arr << "[4 * g]; q.y = " << o.arr << "[4 * g + 1]; q.z = " << o.arr << "[4 * g + 2]; q.w = "
         << o.arr << "[4 * g + 3];\n";
    } else if (ebytes == 4) {
      fn << "        q.x = b200_bits32(" << o.arr << "[4 * g]); q.y = b200_bits32(" << o.arr << "[4 * g + 1]);\n"
         << "        q.z = b200_bits32(" << o.arr << "[4 * g + 2]); q.w = b200_bits32(" << o.arr << "[4 * g + 3]);\n";
    } else {
      const std::string pk = t.prec == Prec::Bfloat16 ? "b200_pack_bf(" : "b200_pack_hf(";
      fn << "        q.x = " << pk << o.arr << "[8 * g], " << o.arr << "[8 * g + 1]);\n"
         << "        q.y = " << pk << o.arr << "[8 * g + 2], " << o.arr << "[8 * g + 3]);\n"
         << "        q.z = " << pk << o.arr << "[8 * g + 4], " << o.arr << "[8 * g + 5]);\n"
         << "        q.w = " << pk << o.arr << "[8 * g + 6], " << o.arr << "[8 * g + 7]);\n";
    }
    fn << "        b200_tile[b200_lane * G + (g ^ B200_STAGE_KEY(b200_lane, G))] = q;\n      }\n";
    return fn.str();
  };
  // Outputs that leave as TMA stores: all of a chunk's tiles are staged (one staging tile each, in
  // groups of B200_STAGING_TILES), made visible to the copy engine with one fence, and issued together
  // by lane 0.  The tiles were read by the previous chunk's copies while this chunk was computed,
  // so the wait before staging is normally over already.
  {
    std::vector<const Out*> tma_outs;
    for (auto& o : outs)
      if (o.tma >= 0) tma_outs.push_back(&o);
    if (!tma_outs.empty()) {
      fn << "  if (b200_es.tma) {\n";
      // groups of at most two outputs (B200_STAGING_TILES is 1 or 2: the group size adapts at compile time of the kernel)
      fn << "    constexpr unsigned int b200_group = B200_STAGING_TILES;\n";
      for (size_t k0 = 0; k0 < tma_outs.size(); ++k0) {
        const Out& o = *tma_outs[k0];
        const int ebytes = prec_bytes(P.tn(o.tn).prec);
        const std::string slot = "(" + std::to_string(k0) + "u % b200_group)";
        fn << "    if (" << slot << " == 0u) {\n"
           << "      if (b200_es.nst) {\n        if (b200_lane == 0) b200_tma_store_read_wait<0>();\n        __syncwarp();\n      }\n      B200_TRE(9);\n    }\n"
           << "    {\n      constexpr int G = B200_EPI_CHUNK / " << (ebytes == 4 ? "4" : "8") << ";\n"
           << "      uint4* b200_tile = b200_stage + " << slot << " * (B200_STAGING_BYTES / 16);\n"
           << sts_code(o) << "    }\n";
        // the group is complete: fence, then lane 0 issues its copies and commits them as one group
        fn << "    if (" << slot << " == b200_group - 1u || " << (k0 + 1 == tma_outs.size() ? "true" : "false") << ") {\n"
           << "      B200_TRE(12);\n      asm volatile(\"fence.proxy.async.shared::cta;\" ::: \"memory\");\n      __syncwarp();\n      B200_TRE(11);\n"
           << "      if (b200_lane == 0) {\n";
        // every output of this group: from the first of the group to k0
        fn << "        constexpr unsigned int b200_first = " << k0 << "u - " << slot << ";\n";
        for (size_t k = 0; k <= k0; ++k)
          fn << "        if (" << k << "u >= b200_first) b200_tma_store_4d_nc(b200_omap" << tma_outs[k]->tma << ", b200_smem_addr(b200_stage + (" << k
             << "u % b200_group) * (B200_STAGING_BYTES / 16)), (int)b200_n0, (int)(b200_m - b200_lane), (int)b200_b1, (int)b200_b0);\n";
        fn << "        b200_tma_commit();\n      }\n      b200_es.nst = 1u;\n      B200_TRE(14);\n    }\n";
      }
      fn << "  }\n";
    }
  }
  for (auto& o : outs) {
    const Tnode& t = P.tn(o.tn);
    const int ebytes = prec_bytes(t.prec);
    const bool vec = o.unit_n && (ebytes == 4 || ebytes == 2);
    const std::string T = Emitter::ctype(t.prec);
    if (o.unit_n) {
      fn << "  {\n    " << T << "* b200_p = b200_row_ok ? (" << t.ident << " + (" << o.row_off << ") + b200_n0) : (" << T << "*)0;\n";
      if (vec) {
        const std::string V = ebytes == 4 ? "4" : "8";  // elements per 16 bytes
        fn << "    constexpr int G = B200_EPI_CHUNK / " << V << ";   // 16-byte groups per row\n";
        if (o.tma >= 0) fn << "    if (!b200_es.tma) {\n";
        else fn << "    {\n";
        fn << "    const bool b200_fast = (b200_n0 + B200_EPI_CHUNK <= b200_N) && __all_sync(0xffffffffu, (((unsigned long long)b200_p) & 15ull) == 0ull);\n"
           << "    if (b200_fast) {\n      uint4* b200_tile = b200_stage;\n"
           << sts_code(o)
           << "      B200_TRE(9);\n      __syncwarp();\n      B200_TRE(14);\n"
           << "#pragma unroll\n      for (int it = 0; it < G; ++it) {\n"
           << "        const unsigned int r = it * (32 / G) + b200_lane / G, c = b200_lane % G;\n"
           << "        const unsigned long long dst = b200_t.r" << o.tn << "[it];\n"
           << "        const uint4 q = b200_stage[r * G + (c ^ B200_STAGE_KEY(r, G))];\n"
           << (reds ? "        if (dst) b200_red_add_v4(dst + (unsigned long long)b200_n0 * "
                    : "        if (dst) *(uint4*)(dst + (unsigned long long)b200_n0 * ")
           << ebytes << (reds ? "ull + 16ull * c, q);\n      }\n" : "ull + 16ull * c) = q;\n      }\n")
           << "      B200_TRE(12);\n      __syncwarp();\n      B200_TRE(11);\n"
           << "    } else if (b200_row_ok) {\n";
      } else {
        fn << "    if (b200_row_ok) {\n";
      }
      fn << "#pragma unroll\n      for (int b200_j = 0; b200_j < B200_EPI_CHUNK; ++b200_j)\n";
      if (reds)
        fn << "        if (b200_n0 + (unsigned int)b200_j < b200_N) atomicAdd(&b200_p[b200_j], "
           << (pair ? "((b200_j & 1) ? " + o.arr + "[b200_j >> 1].y : " + o.arr + "[b200_j >> 1].x)" : o.arr + "[b200_j]") << ");\n";
      else
        fn << "        if (b200_n0 + (unsigned int)b200_j < b200_N) b200_p[b200_j] = "
           << (!pair ? Emitter::store_wrap(t.prec, o.arr + "[b200_j]")
                     : ebytes == 4 ? "((b200_j & 1) ? " + o.arr + "[b200_j >> 1].y : " + o.arr + "[b200_j >> 1].x)"
                                   : "(unsigned short)(" + o.arr + "[b200_j >> 1] >> (16 * (b200_j & 1)))")
           << ";\n";
      fn << "    }\n" << (vec ? "    }\n" : "") << "  }\n";
    } else {
      // general position: recompute the offset per column
      fn << "#pragma unroll\n  for (int b200_j = 0; b200_j < B200_EPI_CHUNK; ++b200_j) {\n"
         << "    const unsigned int b200_n = b200_n0 + (unsigned int)b200_j;\n    if (b200_row_ok && b200_n < b200_N) {\n";
      ep.str("");
      recover(dn, "b200_n");
      fn << ep.str() << "      " << t.ident << "[" << em.offset(o.idcs, t.dims) << "] = " << Emitter::store_wrap(t.prec, o.arr + "[b200_j]") << ";\n    }\n  }\n";
    }
  }
  // row followers: assignments over whole rows, from the register tiles; then the rows' stores
  fn << row_decls;
  if (!row_code.empty()) fn << "  if (b200_row_ok) {\n" << row_code << row_stores << "  }\n";
  fn << final_code;
  fn << "  B200_TRE(15);\n}\n";

  out->kind = Stage::Gemm;
  out->gemm = g;
  out->gemm.epilogue = fn.str();
  out->args = kargs;
  out->writes.clear();
  for (auto& o : outs) out->writes.push_back(o.tn);
  out->writes.insert(out->writes.end(), row_written.begin(), row_written.end());
  out->total = 1;
  out->epi_tiles = (int)outs.size() + n_in_tiles;
  out->epi_out_bytes = 2;
  for (auto& o : outs) out->epi_out_bytes = std::max(out->epi_out_bytes, std::min(4, prec_bytes(P.tn(o.tn).prec)));
  out->epi_params = params_k;
  out->epi_args = args;
  out->epi_prologue = map_prologue;
  out->out_maps = out_maps;
  out->in_maps = in_maps;
  out->row_followers = row_fused;
  out->epi_scratch_bytes = scratch_bytes;
  return true;
}

// Tile shape of a contraction: columns per tile, and whether two CTAs share a 256-row tile.
//
// One tcgen05.mma of K = 16 takes about 128 cycles whether the tile is 16 or 256 columns wide (the
// A operand's 128 rows come out of shared memory at 32 bytes per clock), so a k block costs the
// same ~0.26 us for every shape and wide tiles do more work in it: large problems want the widest
// tile.  A problem of few tiles is different: its time is one tile's main loop plus one tile's
// epilogue, and the epilogue shrinks with the tile (about 3.7 us for 128 rows x 256 columns).  The
// choice minimises  waves x k blocks x 0.26 us + 3.7 us x columns / 256  over the shapes the
// operands allow; 148 SMs are assumed (compilation knows no device).
static void gemm_tile_shape(const GemmPlan& g, int* bn_out, bool* pair_out) {
  const int eb = prec_bytes(g.in_prec);
  const int row_elems = 128 / eb;
  int bn0;
  if (g.n.extent >= 256) bn0 = 256;
  else bn0 = (int)((g.n.extent + 15) / 16 * 16);
  if (!g.b_kmajor) bn0 = (bn0 + row_elems - 1) / row_elems * row_elems;
  if (bn0 > 256) bn0 = 256;
  long long batch = 1;
  for (auto& b : g.batch) batch *= b.extent;
  const double k_blocks = (double)((g.k.extent + row_elems - 1) / row_elems);
  double best = 1e300;
  int best_bn = bn0;
  bool best_pair = false;
  for (int pair = 1; pair >= 0; --pair) {
    for (int bn = bn0; bn >= 16; bn = (bn > 64 ? bn / 2 : 0)) {
      if (bn != bn0 && (bn % 64 != 0 || (!g.b_kmajor && bn % row_elems != 0))) continue;
      // two CTAs per 256 x bn tile need a full pair tile of rows; each CTA stages half of B
      if (pair && !(g.m.extent >= 256 && bn >= 64 && bn % 32 == 0 && (g.b_kmajor || (bn / 2) % row_elems == 0))) continue;
      const long long bm = pair ? 256 : 128, workers = pair ? 74 : 148;
      const long long tiles = batch * ((g.m.extent + bm - 1) / bm) * ((g.n.extent + bn - 1) / bn);
      // few tiles over a long K: several work units per tile, each over a slice of K (gemm_split_k)
      long long split = 1;
      if (g.may_split && tiles * 2 <= workers) split = std::max<long long>(1, std::min<long long>({workers / tiles, (long long)k_blocks / 8, 32ll}));
      const double waves = (double)((tiles * split + workers - 1) / workers);
      // per k block: the MMA floor, or the delivery of the CTA's operand bytes into shared memory
      // (sustained about 64 bytes per clock per SM: single CTAs on 128 x 256 tiles reach 54 % of the
      // tensor peak, CTA pairs, which stage half of B each, 88 %); a CTA pair pays ~0.4 us more
      // set-up (cluster barrier, paired tensor-memory allocation)
      const double kb_us = std::max(0.26, (128.0 + (pair ? bn / 2 : bn)) * 128.0 / 64.0 / 1900.0);
      const double t = waves * (k_blocks / (double)split) * kb_us + 3.7 * bn / 256.0 + (pair ? 0.4 : 0.0);
      if (t < best - 1e-9) {
        best = t;
        best_bn = bn;
        best_pair = pair != 0;
      }
    }
  }
  *bn_out = best_bn;
  *pair_out = best_pair;
}

// Work units per tile.  An accumulation into an fp32 node with few output tiles and a long K (the
// weight gradients: 1024 x 1024 outputs over 8192 rows are 16 pair tiles for 74 pairs) gives
// every tile to several workers, each over a slice of K; their partial tiles meet in the output
// through vector reductions in global memory.  148 SMs are assumed (the compile step knows no device).
static int gemm_split_k(const GemmPlan& g) {
  int bn;
  bool pair;
  gemm_tile_shape(g, &bn, &pair);
  const int bm = pair ? 256 : 128;
  long long tiles = ((g.m.extent + bm - 1) / bm) * ((g.n.extent + bn - 1) / bn);
  for (auto& b : g.batch) tiles *= b.extent;
  const long long workers = pair ? 74 : 148;
  const long long k_blocks = (g.k.extent + (128 / prec_bytes(g.in_prec)) - 1) / (128 / prec_bytes(g.in_prec));
  if (tiles * 2 > workers) return 1;
  long long s = std::min<long long>(workers / tiles, k_blocks / 8);
  return (int)std::max<long long>(1, std::min<long long>(s, 32));
}

std::string gemm_translation_unit(const Program& P, Stage& st, const std::string& kernel_name, const CompileOptions&) {
  GemmPlan& g = st.gemm;
  const int eb = prec_bytes(g.in_prec);
  const int row_elems = 128 / eb;
  int bn;
  bool pair;
  gemm_tile_shape(g, &bn, &pair);
  const int bm = pair ? 256 : 128, bk = row_elems;
  const int umma_k = 32 / eb;
  const int stage_bytes = (128 + (pair ? bn / 2 : bn)) * bk * eb;   // per CTA
  // Epilogue width: the epilogue is a chain of dependent instructions per warp, so it is bound
  // by latency, not issue rate; light epilogues (few register tiles) get 16 warps, which fits
  // the register file at <= 112 registers per thread.
  // columns per epilogue step: more columns = more independent work per thread (the epilogue
  // is latency-bound) and half as many stores to issue; one CTA of 320 threads per SM leaves each
  // thread 200 registers, enough for the register tiles of 32 columns
  int chunk = bn >= 32 ? 32 : 16;
  if (st.row_followers > 0) chunk = bn;   // the whole row in one chunk
  const bool light = false;  // 16 warps measured slower: the register cap (96) makes the epilogue spill
  int epi_warps = light ? 16 : (bn >= 128 ? 8 : 4);
  const int staging = 32 * chunk * st.epi_out_bytes;   // one staging tile
  const int load_tile = st.in_maps.empty() ? 0 : 32 * chunk * st.in_maps[0].elem_bytes;   // a row operand's chunk, per warp
  // outputs that leave as TMA stores alternate between two tiles per warp (the copy engine reads one
  // while the warp fills the other) when that leaves the ring at least four slots
  int staging_tiles = 1;
  if (!st.out_maps.empty() && (227 * 1024 - 1024 - 512 - epi_warps * (staging * 2 + load_tile)) / stage_bytes >= 4) staging_tiles = 2;
  // 227 KB per CTA: ring + alignment slack + barriers + the staging tiles of the epilogue warps
  int stages = (227 * 1024 - 1024 - 512 - epi_warps * (staging * staging_tiles + load_tile)) / stage_bytes;
  if (stages > 8) stages = 8;
  if (stages < 2) stages = 2;
  int tmem_cols = 32;
  while (tmem_cols < 2 * bn) tmem_cols *= 2;
  // instruction descriptor: fp32 accumulate, operand formats, majors, N >> 3, M >> 4
  unsigned int fmt = g.in_prec == Prec::Bfloat16 ? 1u : (g.in_prec == Prec::Half ? 0u : 2u);
  unsigned int idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((g.a_kmajor ? 0u : 1u) << 15) | ((g.b_kmajor ? 0u : 1u) << 16) |
                       ((unsigned int)(bn >> 3) << 17) | ((unsigned int)(bm >> 4) << 24);
  // consecutive tiles walk down this many row tiles before moving to the next column tile
  const int raster = 8;
  const std::string &params = st.epi_params, &args = st.epi_args;
  std::ostringstream o;
  o << kNumericsSource << "\n";
  o << "#define B200_GEMM_NAME " << kernel_name << "\n#define B200_BM " << bm << "\n#define B200_BN " << bn
    << "\n#define B200_BK " << bk << "\n#define B200_UMMA_K " << umma_k << "\n#define B200_ELEM_BYTES " << eb
    << "\n#define B200_STAGES " << stages << "\n#define B200_EPI_WARPS " << epi_warps << "\n#define B200_A_KMAJOR "
    << (g.a_kmajor ? 1 : 0) << "\n#define B200_B_KMAJOR " << (g.b_kmajor ? 1 : 0) << "\n#define B200_IDESC " << idesc
    << "u\n#define B200_TMEM_COLS " << tmem_cols << "\n#define B200_RASTER " << raster << "\n#define B200_CTA_PAIR "
    << (pair ? 1 : 0) << "\n#define B200_SPLITK " << g.split_k << "\n";
  o << "#define B200_EPI_CHUNK " << chunk << "\n#define B200_STAGING_BYTES " << staging << "\n#define B200_STAGING_TILES " << staging_tiles << "\n#define B200_LOAD_TILE_BYTES " << load_tile << "\n";
  o << "#define B200_EPI_PROLOGUE " << [&] { std::string p = st.epi_prologue; for (auto& c : p) if (c == '\n') c = ' '; return p; }() << "\n";
  o << kTcSource << "\n" << g.epilogue << "\n";
  o << "#define B200_EPI_PARAMS " << params << "\n";
  o << "#define B200_EPILOGUE_ROWS b200_epilogue_rows(b200_tiles, b200_b0, b200_b1, b200_m, b200_m < shape.M" << args << ");\n";
  o << "#define B200_EPILOGUE_LOAD b200_epilogue_load(b200_tiles, b200_b0, b200_b1, b200_m, b200_m < shape.M, b200_pn0, shape.N, b200_es" << args << ");\n";
  o << "#define B200_EPILOGUE_ROW b200_epilogue_row(b200_r, b200_b0, b200_b1, b200_m, b200_m < shape.M, b200_n0, shape.N, b200_stage, b200_has_next, b200_next_taddr, b200_tiles, b200_slot, b200_nslots, b200_nx_ok, b200_nx_b0, b200_nx_b1, b200_nx_m, b200_nx_m < shape.M, b200_nx_n0, b200_es" << args << ");\n";
  o << kGemmSource << "\n";
  std::ostringstream note;
  note << "tcgen05 " << (g.in_prec == Prec::Single ? "tf32 " : "") << bm << "x" << bn << "x" << bk << (pair ? " (CTA pair, cta_group::2)" : "") << " stages=" << stages
       << " epi_warps=" << epi_warps << (g.split_k > 1 ? " split_k=" + std::to_string(g.split_k) : std::string())
       << (g.accumulate ? " beta=1" : "")
       << (st.row_followers ? " + " + std::to_string(st.row_followers) + " whole-row assignments in the epilogue" +
                                  (st.epi_scratch_bytes ? " (the last one a grid-wide sum)" : "")
                            : std::string());
  st.note = note.str();
  // remembered for the launcher
  st.block = 64 + 32 * epi_warps;
  st.tile_m = bm;
  st.tile_n = bn;
  st.tile_k = bk;
  st.cta_pair = pair ? 1 : 0;
  st.box_m = 128;
  st.box_n = pair ? bn / 2 : bn;
  st.smem_bytes = stages * stage_bytes + 1024 + 512 + epi_warps * (staging * staging_tiles + load_tile);
  st.epi_chunk = chunk;
  return o.str();
}

}  // namespace b200
