// Launch side of the contraction kernel: TMA tensor maps for the two operands (built once at
// link, when the nodes' addresses are known) and the persistent launch.
#include <cstring>

#include "runtime.hpp"

using namespace b200;

// must match b200_gemm_shape in kernels/gemm_sm100.cuh
struct GemmShape {
  unsigned int M, N, K, B0, B1, a_b0, a_b1, b_b0, b_b1, tiles_m, tiles_n, tma_out;
};

struct GemmLaunch {
  CUtensorMap map_a, map_b;
  std::vector<CUtensorMap> out_maps;   // the epilogue's outputs as TMA store destinations
  std::vector<CUtensorMap> in_maps;    // a row operand of the epilogue as a TMA load source
  GemmShape shape;
  unsigned int grid = 1;
  CUdeviceptr status = 0;
};

static void encode_operand(CUtensorMap* map, CUdeviceptr base, Prec prec, bool kmajor, const GemmDim& mn, int64_t mn_stride,
                           const GemmDim& k, int64_t k_stride, const std::vector<GemmDim>& batch,
                           const std::vector<int64_t>& batch_stride, int tile_mn, int tile_k, int inner_box = 0) {
  const int eb = prec_bytes(prec);
  CUtensorMapDataType dt = prec == Prec::Bfloat16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : prec == Prec::Half   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const int row_elems = 128 / eb;
  cuuint64_t dims[4];
  cuuint64_t strides[3];
  cuuint32_t box[4] = {(cuuint32_t)(inner_box > 0 ? inner_box : row_elems), 1, 1, 1};   // inner_box: a box narrower than one 128-byte swizzle row
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (kmajor) {
    dims[0] = (cuuint64_t)k.extent;
    dims[1] = (cuuint64_t)mn.extent;
    strides[0] = (cuuint64_t)mn_stride * eb;
    box[1] = (cuuint32_t)tile_mn;
  } else {
    dims[0] = (cuuint64_t)mn.extent;
    dims[1] = (cuuint64_t)k.extent;
    strides[0] = (cuuint64_t)k_stride * eb;
    box[1] = (cuuint32_t)tile_k;
  }
  // batch axes: index 2 is the inner one, index 3 the outer one; an operand that does not
  // vary along an axis sees extent 1 there
  const cuuint64_t filler = ((dims[0] * eb + 15) / 16) * 16;
  for (int i = 0; i < 2; ++i) {
    dims[2 + i] = 1;
    strides[1 + i] = filler;
  }
  const int nb = (int)batch.size();
  for (int i = 0; i < nb; ++i) {
    // batch[nb-1] is the innermost
    const int slot = 2 + (nb - 1 - i);
    if (batch_stride[i] != 0) {
      dims[slot] = (cuuint64_t)batch[i].extent;
      strides[slot - 1] = (cuuint64_t)batch_stride[i] * eb;
    }
  }
  // an m/n-major operand of 32-bit elements must lie in shared memory with 32-byte swizzle atoms
  // (see the descriptor notes in kernels/gemm_sm100.cuh); everything else with 16-byte atoms
  const CUtensorMapSwizzle swz = (!kmajor && eb == 4) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  CUresult r = cu().cuTensorMapEncodeTiled_(map, dt, 4, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                            swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw Error(B200_E_UNSUPPORTED, "the operand layout of a contraction cannot be described to the TMA unit (CUresult " +
                                        std::to_string((int)r) + "); compile the routine with gemm=0");
}

GemmLaunch* gemm_prepare(b200_routine* r, int si) {
  const Stage& st = r->code->code.stages[si];
  const GemmPlan& g = st.gemm;
  const Program& P = r->code->code.prog;
  auto ptr = [&](int tn) {
    auto it = r->node_ptr.find(tn);
    if (it == r->node_ptr.end()) throw Error(B200_E_USER, "link: node '" + P.tn(tn).ident + "' has no buffer binding");
    return it->second;
  };
  const int eb = prec_bytes(g.in_prec);
  CUdeviceptr a = ptr(g.a_tn) + (CUdeviceptr)(g.a_off * eb), b = ptr(g.b_tn) + (CUdeviceptr)(g.b_off * eb);
  if ((a & 15) || (b & 15))
    throw Error(B200_E_INVALID, "link: internal error: a contraction stage was kept for operands that are not 16-byte aligned");
  auto* L = new GemmLaunch();
  try {
    std::vector<int64_t> sa, sb;
    for (auto& d : g.batch) { sa.push_back(d.sa); sb.push_back(d.sb); }
    encode_operand(&L->map_a, a, g.in_prec, g.a_kmajor, g.m, g.m.sa, g.k, g.k.sa, g.batch, sa, st.box_m, st.tile_k);
    encode_operand(&L->map_b, b, g.in_prec, g.b_kmajor, g.n, g.n.sb, g.k, g.k.sb, g.batch, sb, st.box_n, st.tile_k);
  } catch (...) {
    delete L;
    throw;
  }
  GemmShape& s = L->shape;
  memset(&s, 0, sizeof s);
  s.M = (unsigned)g.m.extent;
  s.N = (unsigned)g.n.extent;
  s.K = (unsigned)g.k.extent;
  s.B0 = s.B1 = 1;
  s.a_b0 = s.a_b1 = s.b_b0 = s.b_b1 = 0;
  const int nb = (int)g.batch.size();
  if (nb == 2) {
    s.B0 = (unsigned)g.batch[0].extent;
    s.B1 = (unsigned)g.batch[1].extent;
    s.a_b0 = g.batch[0].sa != 0; s.b_b0 = g.batch[0].sb != 0;
    s.a_b1 = g.batch[1].sa != 0; s.b_b1 = g.batch[1].sb != 0;
  } else if (nb == 1) {
    s.B1 = (unsigned)g.batch[0].extent;
    s.a_b1 = g.batch[0].sa != 0; s.b_b1 = g.batch[0].sb != 0;
  }
  // The outputs as TMA store destinations: [n, m, inner batch, outer batch], a box of 32 rows x one
  // epilogue chunk, swizzled like the staging tile (128 / 64 / 32 bytes per row).  If any of them
  // cannot be described (an address that is not 16-byte aligned), the kernel keeps to plain stores.
  s.tma_out = 0;
  if (!st.out_maps.empty()) {
    bool ok = true;
    auto encode = [&](const OutMap& om, CUtensorMap* map) {
      const CUdeviceptr base = ptr(om.tn) + (CUdeviceptr)(om.off * om.elem_bytes);
      const int row_bytes = st.epi_chunk * om.elem_bytes;
      if ((base & 15) || !(row_bytes == 32 || row_bytes == 64 || row_bytes == 128)) return false;
      cuuint64_t dims[4] = {(cuuint64_t)g.n.extent, (cuuint64_t)g.m.extent, 1, 1};
      cuuint64_t strides[3] = {(cuuint64_t)om.m_stride * om.elem_bytes, 0, 0};
      const cuuint64_t filler = ((dims[0] * om.elem_bytes + 15) / 16) * 16;
      strides[1] = strides[2] = filler;
      if (nb == 2) {
        dims[2] = (cuuint64_t)g.batch[1].extent; strides[1] = (cuuint64_t)om.b1_stride * om.elem_bytes;
        dims[3] = (cuuint64_t)g.batch[0].extent; strides[2] = (cuuint64_t)om.b0_stride * om.elem_bytes;
      } else if (nb == 1) {
        dims[2] = (cuuint64_t)g.batch[0].extent; strides[1] = (cuuint64_t)om.b1_stride * om.elem_bytes;
      }
      cuuint32_t box[4] = {(cuuint32_t)st.epi_chunk, 32, 1, 1}, estr[4] = {1, 1, 1, 1};
      const CUtensorMapSwizzle swz = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
      const CUtensorMapDataType dt = om.elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
      return cu().cuTensorMapEncodeTiled_(map, dt, 4, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    L->out_maps.resize(st.out_maps.size());
    for (size_t k = 0; ok && k < st.out_maps.size(); ++k) ok = encode(st.out_maps[k], &L->out_maps[k]);
    L->in_maps.resize(st.in_maps.size());
    for (size_t k = 0; ok && k < st.in_maps.size(); ++k) ok = encode(st.in_maps[k], &L->in_maps[k]);
    if (!ok) {   // placeholders the kernel never uses
      L->out_maps.assign(st.out_maps.size(), L->map_a);
      L->in_maps.assign(st.in_maps.size(), L->map_a);
    }
    s.tma_out = ok ? 1u : 0u;
  } else {
    L->in_maps.assign(st.in_maps.size(), L->map_a);
  }
  s.tiles_m = (s.M + st.tile_m - 1) / st.tile_m;
  s.tiles_n = (s.N + st.tile_n - 1) / st.tile_n;
  unsigned long long tiles = (unsigned long long)s.tiles_m * s.tiles_n * s.B0 * s.B1 * (unsigned long long)(g.split_k > 0 ? g.split_k : 1);
  cu_check(cu().cuFuncSetAttribute_(r->fns[si], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, st.smem_bytes),
           "cuFuncSetAttribute(max dynamic shared memory)");
  if (st.cta_pair) {
    // persistent pairs: as many 2-CTA clusters as the device keeps resident at once
    int clusters = r->dev->sm_count / 2;
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDimX = (unsigned)(r->dev->sm_count / 2 * 2); cfg.gridDimY = 1; cfg.gridDimZ = 1;
    cfg.blockDimX = (unsigned)st.block; cfg.blockDimY = 1; cfg.blockDimZ = 1;
    cfg.sharedMemBytes = (unsigned)st.smem_bytes;
    CUlaunchAttribute attr;
    memset(&attr, 0, sizeof attr);
    attr.id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
    attr.value.clusterDim.x = 2; attr.value.clusterDim.y = 1; attr.value.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int active = 0;
    if (cu().cuOccupancyMaxActiveClusters_(&active, r->fns[si], &cfg) == CUDA_SUCCESS && active > 0 && active < clusters) clusters = active;
    L->grid = 2u * (unsigned)(tiles < (unsigned long long)clusters ? tiles : (unsigned long long)clusters);
  } else {
    L->grid = (unsigned)(tiles < (unsigned long long)r->dev->sm_count ? tiles : (unsigned long long)r->dev->sm_count);
  }
  L->status = r->dev->status_dev;
  return L;
}

void gemm_enqueue(b200_routine* r, int si) {
  const Stage& st = r->code->code.stages[si];
  GemmLaunch* L = r->gemm[si];
  std::vector<void*> args;
  args.push_back(&L->map_a);
  args.push_back(&L->map_b);
  args.push_back(&L->shape);
  args.push_back(&L->status);
  std::vector<CUdeviceptr>& vals = r->arg_values[si];
  for (size_t a = 0; a < vals.size(); ++a) args.push_back(&vals[a]);
  for (auto& m : L->in_maps) args.push_back(&m);
  for (auto& m : L->out_maps) args.push_back(&m);
  launch_kernel(r->dev, r->fns[si], L->grid, (unsigned)st.block, 1, (unsigned)st.smem_bytes, args.data(), "cuLaunchKernelEx(contraction)",
                st.cta_pair ? 2u : 1u);
}

void gemm_release(GemmLaunch* g) { delete g; }

// ---- fused attention stages: three tensor maps (queries and keys k-major, values n-major), one
//      CTA per (batch, head, 128 queries)

// must match b200_attn_shape in kernels/attn_sm100.cuh
struct AttnShape {
  unsigned int S, B0, B1, tiles_s;
};

struct AttnLaunch {
  CUtensorMap map_q, map_k, map_v, map_scores, map_exp, map_w;
  AttnShape shape;
  unsigned int grid = 1;
  CUdeviceptr status = 0;
};

AttnLaunch* attn_prepare(b200_routine* r, int si) {
  const Stage& st = r->code->code.stages[si];
  const AttnPlan& a = st.attn;
  const Program& P = r->code->code.prog;
  auto ptr = [&](int tn) {
    auto it = r->node_ptr.find(tn);
    if (it == r->node_ptr.end()) throw Error(B200_E_USER, "link: node '" + P.tn(tn).ident + "' has no buffer binding");
    return it->second;
  };
  const int eb = prec_bytes(a.in_prec);
  const CUdeviceptr q = ptr(a.q_tn) + (CUdeviceptr)(a.q_off * eb), k = ptr(a.k_tn) + (CUdeviceptr)(a.k_off * eb),
                    v = ptr(a.v_tn) + (CUdeviceptr)(a.v_off * eb);
  if ((q | k | v) & 15)
    throw Error(B200_E_INVALID, "link: internal error: an attention stage was kept for operands that are not 16-byte aligned");
  auto* L = new AttnLaunch();
  try {
    // in the terms of encode_operand: the head dimension is "k" of the first contraction (unit stride);
    // the values are the n-major B operand of the second one (n = head dimension, k = key position)
    std::vector<GemmDim> batch;
    if (a.B0 > 1 || a.B1 > 1) {
      GemmDim b0, b1;
      b0.extent = a.B0;
      b1.extent = a.B1;
      batch = {b0, b1};
    }
    auto strides = [&](int64_t s0, int64_t s1) {
      return batch.empty() ? std::vector<int64_t>{} : std::vector<int64_t>{a.B0 > 1 ? s0 : 0, a.B1 > 1 ? s1 : 0};
    };
    GemmDim qs, ks, ed, td;
    qs.extent = a.S;
    ks.extent = a.T;
    ed.extent = a.E;
    td.extent = a.T;
    encode_operand(&L->map_q, q, a.in_prec, true, qs, a.q_row, ed, 1, batch, strides(a.q_b0, a.q_b1), 128, (int)a.E);
    encode_operand(&L->map_k, k, a.in_prec, true, ks, a.k_row, ed, 1, batch, strides(a.k_b0, a.k_b1), (int)a.T, (int)a.E);
    encode_operand(&L->map_v, v, a.in_prec, false, ed, 1, td, a.v_row, batch, strides(a.v_b0, a.v_b1), (int)a.E, (int)a.T);
    // the row nodes the routine keeps, as destinations of TMA stores: [key, query, inner batch, outer batch],
    // a 32 x 32 box of single-precision values per chunk, a 64 x 128 box of 16-bit weights per block of keys
    auto rows = [&](CUtensorMap* m, const AttnPlan::RowNode& rn, Prec prec, int box_t, int box_s) {
      if (!rn.keep) { *m = L->map_q; return; }   // never used by the kernel
      const CUdeviceptr base = ptr(rn.tn) + (CUdeviceptr)(rn.off * prec_bytes(prec));
      if (base & 15) throw Error(B200_E_INVALID, "link: internal error: an attention stage was kept for a row node that is not 16-byte aligned");
      GemmDim keys, qrows;
      keys.extent = a.T;
      qrows.extent = a.S;
      encode_operand(m, base, prec, true, qrows, rn.row, keys, 1, batch, strides(rn.b0, rn.b1), box_s, box_t, box_t);
    };
    rows(&L->map_scores, a.scores, Prec::Single, 32, 32);
    rows(&L->map_exp, a.exps, Prec::Single, 32, 32);
    rows(&L->map_w, a.weights, a.in_prec, 64, 128);
  } catch (...) {
    delete L;
    throw;
  }
  L->shape.S = (unsigned)a.S;
  L->shape.B0 = (unsigned)a.B0;
  L->shape.B1 = (unsigned)a.B1;
  L->shape.tiles_s = (unsigned)((a.S + 127) / 128);
  L->grid = L->shape.tiles_s * L->shape.B0 * L->shape.B1;
  cu_check(cu().cuFuncSetAttribute_(r->fns[si], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, st.smem_bytes),
           "cuFuncSetAttribute(max dynamic shared memory)");
  L->status = r->dev->status_dev;
  return L;
}

void attn_enqueue(b200_routine* r, int si) {
  const Stage& st = r->code->code.stages[si];
  AttnLaunch* L = r->attn[si];
  std::vector<void*> args;
  args.push_back(&L->map_q);
  args.push_back(&L->map_k);
  args.push_back(&L->map_v);
  args.push_back(&L->map_scores);
  args.push_back(&L->map_exp);
  args.push_back(&L->map_w);
  args.push_back(&L->shape);
  args.push_back(&L->status);
  std::vector<CUdeviceptr>& vals = r->arg_values[si];
  for (size_t a = 0; a < vals.size(); ++a) args.push_back(&vals[a]);
  launch_kernel(r->dev, r->fns[si], L->grid, (unsigned)st.block, 1, (unsigned)st.smem_bytes, args.data(), "cuLaunchKernelEx(attention)", 1u);
}

void attn_release(AttnLaunch* a) { delete a; }
