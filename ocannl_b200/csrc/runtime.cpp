// Linking and launching of compiled routines.
//
// `link` binds every in-context node of the routine to {pool, offset}
// (`Lowered_backend.link`, arrayjit/lib/backend_impl.ml:334-367; the cuda backend resolves the
// same pairs at each launch, arrayjit/lib/cuda_backend.ml:1005-1009) and loads the routine's
// machine code.  `launch` enqueues the stages on the device stream; static index values
// travel through a small device table so that a captured CUDA graph stays valid when they
// change between runs.
#include "runtime.hpp"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

using namespace b200;

static const size_t kRing = 512;

CUdeviceptr b200_dev::address(int pool_id, size_t offset, size_t bytes) {
  std::lock_guard<std::mutex> g(mu);
  auto it = pools.find(pool_id);
  if (it == pools.end()) throw Error(B200_E_INVALID, "unknown pool id " + std::to_string(pool_id));
  if (offset > it->second.bytes || bytes > it->second.bytes - offset)
    throw Error(B200_E_INVALID, "range [" + std::to_string(offset) + ", +" + std::to_string(bytes) + ") exceeds pool " +
                                    std::to_string(pool_id) + " of " + std::to_string(it->second.bytes) + " bytes");
  return it->second.ptr + offset;
}

void b200_dev::check_status() {
  if (status_host && getenv("B200_TRACE")) {
    fprintf(stderr, "[b200 trace] ns since CTA 0 start: setup %u, first loads issued %u, producer done %u, first operands %u, "
                    "tile0 mma issued %u, tile1 mma issued %u, epi0 begin %u end %u, epi1 begin %u end %u, all done %u\n"
                    "[b200 trace] epilogue cycles of warp 2 by phase: accumulator wait %u, tmem load wait %u, operand loads + "
                    "compute %u, staging %u, stores %u, release %u\n",
            status_host[2], status_host[3], status_host[4], status_host[5], status_host[6], status_host[7], status_host[8],
            status_host[9], status_host[10], status_host[11], status_host[12], status_host[16 + 3], status_host[16 + 4],
            status_host[16 + 13], status_host[16 + 14], status_host[16 + 15], status_host[16 + 5]);
    fprintf(stderr, "[b200 trace] epilogue store blocks, cycles: next-chunk loads %u, staging writes %u, first warp sync %u, staged reads + global stores %u, "
                    "second warp sync %u\n",
            status_host[16 + 10], status_host[16 + 9], status_host[16 + 14], status_host[16 + 12], status_host[16 + 11]);
    fprintf(stderr, "[b200 trace] attention CTA, ns since its start: setup %u, q and k landed %u, scores ready %u, pass 1 %u, pass 2 %u, "
                    "pass 3 %u, second mma issued %u, weights copied %u, output ready %u, stored %u\n",
            status_host[40], status_host[41], status_host[42], status_host[43], status_host[44], status_host[45], status_host[46],
            status_host[47], status_host[48], status_host[49]);
  }
  if (status_host && status_host[0] != 0) {
    unsigned int code = status_host[0], where = status_host[1];
    const unsigned long long index = (unsigned long long)status_host[2] | ((unsigned long long)status_host[3] << 32);
    status_host[0] = 0;
    status_host[1] = 0;
    if (code == 2u)
      throw Error(B200_E_DEVICE, "range-checked build: an access to node id " + std::to_string(where) + " at element " +
                                     std::to_string(index) + " lies outside the node (skipped)");
    throw Error(B200_E_DEVICE, "a kernel gave up a bounded wait (code " + std::to_string(code) + ", site " +
                                   std::to_string(where) + ")");
  }
}

// Which stages of `c` cannot run in the compiled form at these addresses?  Pair-form generic
// stages read and write 8-byte words; the contraction kernel's tensor maps want 16-byte operand
// bases.  The reference's allocator aligns a node to its element size only
// (`plan_pool_segments`, arrayjit/lib/backends.ml:22-51), so such bindings are legitimate: the
// statements behind those stages are re-planned without the demanding form.
static bool misaligned_stages(const b200_code* c, const std::map<int, CUdeviceptr>& param_ptr, std::set<int>* no_pairs_at,
                              std::set<int>* no_gemm_at) {
  bool any = false;
  const Program& P = c->code.prog;
  auto at = [&](int tn) -> CUdeviceptr {
    auto it = param_ptr.find(tn);
    return it == param_ptr.end() ? 0 : it->second;   // routine-local nodes sit at 256-byte multiples
  };
  for (auto& st : c->code.stages) {
    if (st.kind == Stage::Generic && st.min_align > 1) {
      bool bad = false;
      for (auto& a : st.args)
        if (a.kind == KArg::Node && (at(a.tn) % (CUdeviceptr)st.min_align) != 0) bad = true;
      if (bad)
        for (int o : st.origins) any |= no_pairs_at->insert(o).second;
    } else if (st.kind == Stage::Gemm) {
      const int eb = prec_bytes(st.gemm.in_prec);
      const CUdeviceptr a = at(st.gemm.a_tn) + (CUdeviceptr)(st.gemm.a_off * eb), b = at(st.gemm.b_tn) + (CUdeviceptr)(st.gemm.b_off * eb);
      (void)P;
      if ((a & 15) || (b & 15))
        for (int o : st.origins) any |= no_gemm_at->insert(o).second;
    } else if (st.kind == Stage::Attn) {
      // tensor maps over the queries, keys and values; 16-byte row stores into every node it writes
      bool bad = ((at(st.attn.q_tn) | at(st.attn.k_tn) | at(st.attn.v_tn)) & 15) != 0;
      for (auto& a : st.args)
        if (a.kind == KArg::Node && (at(a.tn) & 15) != 0) bad = true;
      if (bad)
        for (int o : st.origins) any |= no_gemm_at->insert(o).second;
    }
  }
  return any;
}

void b200_routine::link(b200_dev* d, b200_code* c, const b200_binding* b, int n) {
  dev = d;
  requested = c;
  std::map<int, const b200_binding*> bind;
  for (int i = 0; i < n; ++i) {
    bind[b[i].tn_id] = &b[i];
    pools_used.insert(b[i].pool_id);
  }
  std::map<int, CUdeviceptr> param_ptr;
  for (auto& t : c->code.prog.tnodes) {
    if (!t.is_param()) continue;
    auto it = bind.find(t.id);
    if (it == bind.end()) continue;  // checked per stage below: only nodes a stage uses are required
    if (it->second->offset % (uint64_t)prec_bytes(t.prec) != 0)
      throw Error(B200_E_INVALID, "link: node '" + t.ident + "' is bound at offset " + std::to_string(it->second->offset) +
                                      ", not a multiple of its element size");
    param_ptr[t.id] = d->address(it->second->pool_id, it->second->offset, (size_t)t.bytes());
  }
  {
    std::set<int> no_pairs_at = c->opt.no_pairs_at, no_gemm_at = c->opt.no_gemm_at;
    b200_code* use = c;
    for (int round = 0; round < 4 && misaligned_stages(use, param_ptr, &no_pairs_at, &no_gemm_at); ++round)
      use = c->variant(no_pairs_at, no_gemm_at);
    c = use;
  }
  code = c;
  const Program& P = c->code.prog;

  // routine-local nodes live in a scratch slab owned by the routine
  size_t off = 0;
  std::map<int, size_t> local_off;
  for (int id : c->code.local_nodes) {
    const Tnode& t = P.tn(id);
    local_off[id] = off;
    if (t.zero_init) scratch_zero.push_back({off, (size_t)t.bytes()});
    off += ((size_t)t.bytes() + 255) & ~(size_t)255;
  }
  // neighbouring zero ranges become one memset (the padding between nodes may be cleared too)
  {
    std::vector<std::pair<size_t, size_t>> merged;
    for (auto& z : scratch_zero) {
      if (!merged.empty() && merged.back().first + merged.back().second + 256 >= z.first)
        merged.back().second = z.first + z.second - merged.back().first;
      else
        merged.push_back(z);
    }
    scratch_zero.swap(merged);
  }
  const size_t reduce_off = off;
  off += c->code.reduce_scratch_bytes;
  scratch_bytes = off;
  if (scratch_bytes) {
    cu_check(cu().cuMemAlloc_(&scratch, scratch_bytes), "cuMemAlloc(scratch)");
    // the tickets of grid-wide reductions start at zero (each kernel resets its own afterwards)
    if (c->code.reduce_scratch_bytes)
      cu_check(cu().cuMemsetD8Async_(scratch + reduce_off, 0, c->code.reduce_scratch_bytes, d->stream), "cuMemsetD8Async(reduce scratch)");
  }

  for (auto& t : P.tnodes) {
    if (t.mode == Mode::Local) node_ptr[t.id] = scratch + local_off[t.id];
    else if (param_ptr.count(t.id)) node_ptr[t.id] = param_ptr[t.id];
  }

  if (!P.statics.empty()) {
    cu_check(cu().cuMemAlloc_(&statics_dev, 256 + 4 * P.statics.size()), "cuMemAlloc(statics)");
    void* hp = nullptr;
    cu_check(cu().cuMemHostAlloc_(&hp, kRing * 4 * P.statics.size(), 0), "cuMemHostAlloc(statics)");
    statics_ring = (unsigned int*)hp;
  }

  if (c->cubin) cu_check(cu().cuModuleLoadData_(&module, c->cubin->data()), "cuModuleLoadData");
  const size_t ns = c->code.stages.size();
  fns.assign(ns, nullptr);
  arg_values.assign(ns, {});
  gemm.assign(ns, nullptr);
  attn.assign(ns, nullptr);
  gemm_modules.assign(ns, nullptr);
  for (size_t i = 0; i < ns; ++i) {
    const Stage& st = c->code.stages[i];
    if (st.kind == Stage::Memset) {
      if (!node_ptr.count(st.memset_tn))
        throw Error(B200_E_USER, "link: node '" + P.tn(st.memset_tn).ident + "' has no buffer binding");
      continue;
    }
    for (auto& a : st.args) {
      if (a.kind == KArg::Node) {
        auto it = node_ptr.find(a.tn);
        if (it == node_ptr.end()) throw Error(B200_E_USER, "link: node '" + P.tn(a.tn).ident + "' has no buffer binding");
        if (st.min_align > 1 && (it->second % (CUdeviceptr)st.min_align) != 0)
          throw Error(B200_E_INVALID, "link: internal error: stage '" + st.kernel + "' kept a form that needs " +
                                          std::to_string(st.min_align) + "-byte alignment for node '" + P.tn(a.tn).ident + "'");
        arg_values[i].push_back(it->second);
      } else if (a.kind == KArg::Status) {
        arg_values[i].push_back(dev->status_dev);
      } else if (a.kind == KArg::Statics) {
        arg_values[i].push_back(statics_dev);
      } else if (a.kind == KArg::Scratch) {
        arg_values[i].push_back(scratch + reduce_off + (size_t)a.tn);
      } else {
        arg_values[i].push_back(0);  // merge buffer: resolved at launch (pool 0 may be re-allocated)
        reads_merge = true;
      }
    }
    if (st.kind == Stage::Generic) {
      cu_check(cu().cuModuleGetFunction_(&fns[i], module, st.kernel.c_str()), "cuModuleGetFunction");
    } else {
      cu_check(cu().cuModuleLoadData_(&gemm_modules[i], c->gemm_cubins[i]->data()), "cuModuleLoadData(gemm)");
      cu_check(cu().cuModuleGetFunction_(&fns[i], gemm_modules[i], st.kernel.c_str()), "cuModuleGetFunction(gemm)");
      if (st.kind == Stage::Attn) attn[i] = attn_prepare(this, (int)i);
      else gemm[i] = gemm_prepare(this, (int)i);
    }
  }
}

// One kernel launch.  Every kernel of this library releases its dependents at entry and waits for
// the grids before it (griddepcontrol) ahead of its first access to memory, so a launch may be
// marked for programmatic stream serialisation: the next kernel's blocks are placed, and run their
// set-up, while the tail of the previous kernel drains.  B200_PDL=0 turns the marking off.
void launch_kernel(b200_dev* dev, CUfunction fn, unsigned grid, unsigned bx, unsigned by, unsigned smem, void** args,
                   const char* what, unsigned cluster) {
  static const bool pdl = [] {
    const char* e = getenv("B200_PDL");
    return !(e && e[0] == '0');
  }();
  CUlaunchConfig cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDimX = grid; cfg.gridDimY = 1; cfg.gridDimZ = 1;
  cfg.blockDimX = bx; cfg.blockDimY = by; cfg.blockDimZ = 1;
  cfg.sharedMemBytes = smem;
  cfg.hStream = dev->stream;
  CUlaunchAttribute attr[2];
  memset(attr, 0, sizeof attr);
  unsigned n = 0;
  if (cluster > 1) {
    attr[n].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
    attr[n].value.clusterDim.x = cluster; attr[n].value.clusterDim.y = 1; attr[n].value.clusterDim.z = 1;
    ++n;
  }
  if (pdl) {
    attr[n].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
    attr[n].value.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cu_check(cu().cuLaunchKernelEx_(&cfg, fn, args, nullptr), what);
}

static void nccl_ok(ncclResult_t r, const char* what) {
  if (r != ncclSuccess) throw Error((int)r, std::string(what) + ": " + nccl().ncclGetErrorString_(r));
}

// The bucket's allreduce on the communicator's stream, ordered after everything queued on the
// compute stream so far; `done` marks its end for the join at the end of the routine.  Inside a
// stream capture the same calls fork the communicator's stream into the graph.
void b200_routine::enqueue_bucket(OverlapBucket& b) {
  b200_comm* c = overlap_comm;
  const size_t esz = b.dtype == B200_F32 ? 4 : 2;
  CUdeviceptr p = dev->address(b.pool_id, b.offset, b.count * esz);
  cu_check(cu().cuEventRecord_(b.ready, dev->stream), "cuEventRecord(bucket ready)");
  cu_check(cu().cuStreamWaitEvent_(c->stream, b.ready, 0), "cuStreamWaitEvent(bucket ready)");
  nccl_ok(nccl().ncclAllReduce_((const void*)p, (void*)p, b.count, b.dtype == B200_F32 ? ncclFloat32 : ncclBfloat16,
                                b.op == B200_SUM ? ncclSum : ncclAvg, c->comm, (cudaStream_t)c->stream),
          "ncclAllReduce(bucket)");
  cu_check(cu().cuEventRecord_(b.done, c->stream), "cuEventRecord(bucket done)");
}

void b200_routine::enqueue_stages() {
  const Program& P = code->code.prog;
  for (auto& z : scratch_zero)
    cu_check(cu().cuMemsetD8Async_(scratch + z.first, 0, z.second, dev->stream), "cuMemsetD8Async(scratch)");
  if (profiling && stage_events.size() != code->code.stages.size()) stage_events.assign(code->code.stages.size(), {});
  struct Timer {
    b200_routine* r;
    size_t i;
    CUevent a = nullptr, b = nullptr;
    Timer(b200_routine* r_, size_t i_) : r(r_), i(i_) {
      if (!r->profiling) return;
      cu_check(cu().cuEventCreate_(&a, CU_EVENT_DEFAULT), "cuEventCreate");
      cu_check(cu().cuEventCreate_(&b, CU_EVENT_DEFAULT), "cuEventCreate");
      cu_check(cu().cuEventRecord_(a, r->dev->stream), "cuEventRecord");
    }
    ~Timer() {
      if (!a) return;
      cu().cuEventRecord_(b, r->dev->stream);
      r->stage_events[i].push_back({a, b});
    }
  };
  // buckets no stage writes into are reduced first; the others as soon as their last writer is queued
  for (auto& b : buckets)
    if (b.after_stage < 0) enqueue_bucket(b);
  // queues stage i (a clear may take the clears that follow along, advancing i)
  auto queue_stage = [&](size_t& i) {
    const Stage& st = code->code.stages[i];
    Timer timer(this, i);
    if (st.kind == Stage::Memset) {
      // zero_outs of nodes that lie back to back in memory (parameter gradients allocated as one
      // range) become one clear; nothing between two nodes is touched unless they are adjacent
      CUdeviceptr at = node_ptr[st.memset_tn];
      size_t bytes = (size_t)P.tn(st.memset_tn).bytes();
      auto fires_after = [&](size_t k) {
        for (auto& b : buckets)
          if (b.after_stage == (int)k) return true;
        return false;
      };
      while (!profiling && !fires_after(i) && i + 1 < code->code.stages.size() && code->code.stages[i + 1].kind == Stage::Memset) {
        const int next_tn = code->code.stages[i + 1].memset_tn;
        const CUdeviceptr next_at = node_ptr[next_tn];
        const size_t next_bytes = (size_t)P.tn(next_tn).bytes();
        if (next_at == at + bytes) bytes += next_bytes;
        else if (next_at + next_bytes == at) { at = next_at; bytes += next_bytes; }
        else break;
        ++i;
      }
      cu_check(cu().cuMemsetD8Async_(at, 0, bytes, dev->stream), "cuMemsetD8Async");
      return;
    }
    if (st.kind == Stage::Generic && st.total <= 0) return;
    if (st.kind == Stage::Gemm || st.kind == Stage::Attn) {
      if (st.kind == Stage::Gemm) gemm_enqueue(this, (int)i);
      else attn_enqueue(this, (int)i);
      dev->n_launches++;
      return;
    }
    std::vector<CUdeviceptr>& vals = arg_values[i];
    for (size_t a = 0; a < st.args.size(); ++a)
      if (st.args[a].kind == KArg::Merge) vals[a] = dev->address(0, 0, (size_t)P.tn(P.merge_node).bytes());
    std::vector<void*> args(vals.size());
    for (size_t a = 0; a < vals.size(); ++a) args[a] = &vals[a];
    long long threads = st.coop ? st.total * st.coop : st.total;
    long long blocks = (threads + st.block - 1) / st.block;
    long long cap = (long long)dev->sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (st.block_y > 1) blocks = std::min<long long>(cap, (st.total + st.block - 1) / st.block);
    if (st.grid_override > 0) blocks = st.grid_override;
    launch_kernel(dev, fns[i], (unsigned)blocks, (unsigned)st.block, (unsigned)st.block_y, 0, args.data(), "cuLaunchKernelEx");
    dev->n_launches++;
  };
  for (size_t i = 0; i < code->code.stages.size(); ++i) {
    queue_stage(i);
    for (auto& b : buckets)
      if (b.after_stage == (int)i) enqueue_bucket(b);
  }
  // whatever follows the routine on the compute stream (the optimizer step) sees the reduced ranges
  for (auto& b : buckets) cu_check(cu().cuStreamWaitEvent_(dev->stream, b.done, 0), "cuStreamWaitEvent(bucket done)");
}

void b200_routine::launch(const int64_t* static_idx, int n_static) {
  const Program& P = code->code.prog;
  if (n_static != (int)P.statics.size())
    throw Error(B200_E_USER, "routine '" + P.name + "' takes " + std::to_string(P.statics.size()) + " static indices, got " +
                                 std::to_string(n_static));
  if (n_static > 0) {
    bool changed = !statics_valid;
    for (int i = 0; i < n_static; ++i) {
      long long v = static_idx[i];
      if (v < 0) throw Error(B200_E_USER, "static index " + P.statics[i].sym + " is negative: " + std::to_string(v));
      if (P.statics[i].range >= 0 && v >= P.statics[i].range)
        throw Error(B200_E_USER, "static index " + P.statics[i].sym + " is too big: " + std::to_string(v) + " >= " +
                                     std::to_string(P.statics[i].range));
      if (v > 0xffffffffLL) throw Error(B200_E_USER, "static index " + P.statics[i].sym + " does not fit 32 bits");
      if (!statics_valid || last_statics[i] != v) changed = true;
    }
    if (changed) {
      if (ring_pos == kRing) {  // staging slots may still be in flight: drain before reuse
        cu_check(cu().cuStreamSynchronize_(dev->stream), "cuStreamSynchronize");
        ring_pos = 0;
      }
      unsigned int* slot = statics_ring + ring_pos * n_static;
      ++ring_pos;
      last_statics.assign(static_idx, static_idx + n_static);
      for (int i = 0; i < n_static; ++i) slot[i] = (unsigned int)static_idx[i];
      cu_check(cu().cuMemcpyHtoDAsync_(statics_dev, slot, 4 * (size_t)n_static, dev->stream), "cuMemcpyHtoDAsync(statics)");
      statics_valid = true;
    }
  }
  // The first run with collectives attached is queued directly: NCCL sets up the connections a
  // collective needs the first time it runs (allocations, exchanges with the peers), which must
  // not happen inside a stream capture.  Later runs capture and replay.
  const bool capture_ok = buckets.empty() || overlap_warm;
  if (!buckets.empty()) overlap_warm = true;
  if (want_graph && !profiling && capture_ok) {
    if (graph && reads_merge && graph_merge_epoch != dev->merge_epoch) {
      // the merge buffer moved since the capture (`b200_merge_copy` grew pool 0): the graph holds
      // the old address
      cu().cuGraphExecDestroy_(graph);
      graph = nullptr;
    }
    if (!graph) {
      graph_merge_epoch = dev->merge_epoch;
      CUgraph g = nullptr;
      cu_check(cu().cuStreamBeginCapture_(dev->stream, CU_STREAM_CAPTURE_MODE_THREAD_LOCAL), "cuStreamBeginCapture");
      try {
        enqueue_stages();
      } catch (...) {
        cu().cuStreamEndCapture_(dev->stream, &g);
        if (g) cu().cuGraphDestroy_(g);
        throw;
      }
      cu_check(cu().cuStreamEndCapture_(dev->stream, &g), "cuStreamEndCapture");
      CUresult r = cu().cuGraphInstantiateWithFlags_(&graph, g, 0);
      cu().cuGraphDestroy_(g);
      cu_check(r, "cuGraphInstantiate");
    }
    cu_check(cu().cuGraphLaunch_(graph, dev->stream), "cuGraphLaunch");
    dev->n_graph_launches++;
    for (auto& s : code->code.stages) dev->n_launches += s.kind != Stage::Memset;
    return;
  }
  enqueue_stages();
}

void b200_routine::set_graph(bool on) {
  want_graph = on;
  if (!on && graph) {
    cu().cuGraphExecDestroy_(graph);
    graph = nullptr;
  }
}

void b200_routine::stage_time(int stage, float* total_ms, int* runs) {
  if (stage < 0 || stage >= (int)code->code.stages.size()) throw Error(B200_E_INVALID, "stage out of range");
  *total_ms = 0;
  *runs = 0;
  if ((size_t)stage >= stage_events.size()) return;
  for (auto& e : stage_events[stage]) {
    cu_check(cu().cuEventSynchronize_(e.second), "cuEventSynchronize");
    float ms = 0;
    cu_check(cu().cuEventElapsedTime_(&ms, e.first, e.second), "cuEventElapsedTime");
    *total_ms += ms;
    ++*runs;
  }
}

void b200_routine::destroy() {
  if (dev) cu().cuStreamSynchronize_(dev->stream);
  if (overlap_comm) overlap_comm->routines.erase(this);
  overlap_comm = nullptr;
  for (auto& v : stage_events)
    for (auto& e : v) {
      cu().cuEventDestroy_(e.first);
      cu().cuEventDestroy_(e.second);
    }
  stage_events.clear();
  if (graph) cu().cuGraphExecDestroy_(graph);
  for (auto& b : buckets) {
    if (b.ready) cu().cuEventDestroy_(b.ready);
    if (b.done) cu().cuEventDestroy_(b.done);
  }
  buckets.clear();
  for (auto* g : gemm) gemm_release(g);
  for (auto* a : attn) attn_release(a);
  for (auto m : gemm_modules)
    if (m) cu().cuModuleUnload_(m);
  if (module) cu().cuModuleUnload_(module);
  if (scratch) cu().cuMemFree_(scratch);
  if (statics_dev) cu().cuMemFree_(statics_dev);
  if (statics_ring) cu().cuMemFreeHost_(statics_ring);
  graph = nullptr;
  module = nullptr;
  scratch = 0;
  statics_dev = 0;
  statics_ring = nullptr;
}
