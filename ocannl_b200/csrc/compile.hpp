// Device-independent compilation of a routine: the b200ir body is cut into stages, each
// stage is classified (memset / generic loop nest / dense contraction) and CUDA source is
// generated for it.  Mirrors the role of `Lowered_backend.compile`
// (arrayjit/lib/backend_impl.ml:334-367): no device or context is touched here.
#pragma once
#include <set>
#include <string>
#include <vector>

#include "ir.hpp"

namespace b200 {

struct LoopDim {
  std::string sym;
  int64_t from = 0, to = 0;  // inclusive, as in Low_level.For_loop
  int64_t extent() const { return to >= from ? to - from + 1 : 0; }
};

// One kernel argument: a tensor node pointer (in-context node, or a routine-local node that
// lives in the routine's scratch slab), the static-index table, or the merge buffer.
struct KArg {
  enum Kind { Node, Statics, Merge, Scratch, Status } kind;   // Status: the device status word (range-checked builds)
  int tn = -1;  // node id; for Scratch: byte offset into the routine's reduction scratch
};

// A dense contraction recognised in the loop nest, in GEMM terms:
//   D[batch, m, n] (+)= sum_k A[batch, m, k] * B[batch, n, k]
// Every symbol group carries its extent and the element stride it has in each tensor.
struct GemmDim {
  int64_t extent = 1;
  int64_t sa = 0, sb = 0, sd = 0;  // element strides in A, B and the output
};
struct GemmPlan {
  int a_tn = -1, b_tn = -1, d_tn = -1;  // d_tn: the node the epilogue's Set writes
  GemmDim m, n, k;
  std::vector<GemmDim> batch;        // outermost first, at most 2
  int64_t a_off = 0, b_off = 0;      // constant element offsets (fixed indices)
  bool a_kmajor = true, b_kmajor = true;
  bool accumulate = false;           // beta = 1: add to the existing output (form B without zero_out)
  Prec in_prec = Prec::Bfloat16;     // operand precision (bf16 / half; single runs as tf32)
  bool may_split = false;            // an fp32 accumulation whose K may be cut into work units (see split_k)
  int split_k = 1;                   // >1: that many work units per tile, each over a slice of K, added with vector reds
  std::string epilogue;              // generated device code, see codegen
  double flops() const;
};

// The fused attention chain (attn_match.cpp): operand layouts for the three tensor maps and the
// generated device functions.  Strides are in elements.
struct AttnPlan {
  int q_tn = -1, k_tn = -1, v_tn = -1;
  int64_t q_off = 0, k_off = 0, v_off = 0;
  int64_t S = 0, T = 0, E = 0, B0 = 1, B1 = 1;   // queries, keys, head dimension, batch extents (outer, inner)
  int64_t q_row = 0, k_row = 0, v_row = 0;      // stride of the query / key position
  int64_t q_b0 = 0, q_b1 = 0, k_b0 = 0, k_b1 = 0, v_b0 = 0, v_b1 = 0;
  Prec in_prec = Prec::Bfloat16;
  int out_bytes = 2;
  int n_cond = 0;          // operands of the score expression handed to the kernel as one bit per element
  std::vector<int> cond_tns;   // their nodes, in the order of the stage's scratch arguments (the packed bits)
  int n_tiles = 0;         // operands of the score expression loaded through the staging tile
  // the three row nodes (scores, exponentials, weights): written by TMA stores when the routine keeps them
  struct RowNode {
    bool keep = false;
    int tn = -1;
    int64_t off = 0, row = 0, b0 = 0, b1 = 0;   // element offset and strides of (query position, outer batch, inner batch)
  };
  RowNode scores, exps, weights;
  std::string code;
};

// An output of a contraction epilogue described to the TMA unit: [n, m, inner batch, outer batch].
// Offsets and strides in elements.
struct OutMap {
  int tn = -1;
  int64_t off = 0, m_stride = 0, b0_stride = 0, b1_stride = 0;
  int elem_bytes = 4;
};

struct Stage {
  enum Kind { Memset, Generic, Gemm, Attn } kind = Generic;
  bool own_module() const { return kind == Gemm || kind == Attn; }   // compiled as a translation unit of its own
  int memset_tn = -1;
  std::string kernel;            // kernel symbol in the routine's module
  std::vector<KArg> args;
  std::vector<LoopDim> par, ser;
  int64_t total = 1;             // parallel iterations
  int block = 256;
  int block_y = 1;               // >1: two-dimensional block (serial loops split over y)
  int coop = 0;                  // >0: lanes cooperating on one output element (row reductions)
  int grid_override = 0;         // >0: launch exactly this many blocks (first pass of a grid-wide reduction)
  GemmPlan gemm;
  AttnPlan attn;
  std::string gemm_source;       // full translation unit of this stage's contraction kernel
  std::string epi_params, epi_args;  // epilogue plumbing: extra kernel parameters / call arguments
  std::string epi_prologue;          // declarations at the top of the kernel's epilogue role (pointers to the output maps)
  std::vector<OutMap> out_maps;      // outputs that leave as TMA stores, in the order of the kernel's map parameters
  std::vector<OutMap> in_maps;       // a row operand of the epilogue that arrives by TMA loads (its map precedes the outputs')
  int epi_chunk = 32;                // columns per epilogue step (the inner box of the output maps)
  int tile_m = 0, tile_n = 0, tile_k = 0;
  int min_align = 0;             // >0: every node the stage touches must be bound at a multiple of this many bytes
  int cta_pair = 0;              // 1: two CTAs of a cluster share one tile_m x tile_n tile (cta_group::2)
  int box_m = 0, box_n = 0;      // rows of A / B one CTA stages per k block (the TMA boxes)
  int smem_bytes = 0;            // dynamic shared memory of the contraction kernel
  int epi_out_bytes = 4;         // widest element the epilogue stores through the staging tile (2 or 4)
  int epi_tiles = 0;             // register tiles (inputs + outputs) the epilogue keeps per chunk
  int row_followers = 0;         // assignments over whole output rows evaluated in the epilogue (the tile is one chunk wide)
  size_t epi_scratch_bytes = 0;  // >0: the epilogue ends in a grid-wide sum; per-warp partials + ticket live in scratch
  std::string note;              // human-readable classification, for debug info
  std::vector<int> origins;      // indices of the routine's top-level statements this stage runs
  std::vector<int> writes;       // nodes the stage writes
};

// A loop nest that follows a contraction and may be folded into its epilogue.
struct Follower {
  std::vector<LoopDim> nest;
  const Stmt* set = nullptr;
};

struct Code {
  Program prog;
  std::vector<Stage> stages;
  std::string source;            // one translation unit holding every generic kernel
  std::vector<int> local_nodes;  // routine-local nodes that need scratch
  size_t reduce_scratch_bytes = 0;  // partial results of grid-wide reductions
  std::string describe() const;  // JSON-ish summary for b200_code_info
};

struct CompileOptions {
  bool enable_gemm = true;
  bool enable_coop = true;
  bool enable_fuse = true;   // several small stages in one single-block kernel
  bool enable_splitk = true; // few-tile accumulations split K over the idle SMs (fp32 atomic adds: order not fixed)
  bool enable_pairs = true;  // contraction epilogues over pairs of columns with packed 16-bit arithmetic
  bool enable_attn = true;   // the attention chain as one fused kernel
  bool enable_tf32 = true;   // single-precision operands of a contraction go through the tensor cores as tf32
  bool large_models = false;
  // Range-checked build: every access a generated kernel makes to a node is checked against the node's
  // size; an access outside it is skipped and reported through the device status word.  Implies the
  // generic kernels (no tensor-core stages, no pair or register-row forms).
  bool bounds = false;
  // Top-level statements (by index) that must not use the forms with alignment demands: the pair
  // form of generic stages (8-byte accesses) / the TMA-fed contraction kernel (16-byte operand
  // bases).  Filled when a routine is linked to buffers at element-size-aligned offsets, as
  // `Raise_backend.allocate_delta` hands them out (arrayjit/lib/backends.ml:529-614).
  std::set<int> no_pairs_at, no_gemm_at;
};

Code compile_program(Program prog, const CompileOptions& opt);

// The numeric helper prelude shared by every generated kernel (embedded at build time).
extern const char* kNumericsSource;
extern const char* kTcSource;
extern const char* kGemmSource;
extern const char* kAttnSource;

}  // namespace b200
