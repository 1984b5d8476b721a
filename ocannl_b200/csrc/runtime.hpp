// Run-time objects behind the C ABI: devices with their pool tables and stream, events,
// compiled code and linked routines.
#pragma once
#include <map>
#include <memory>
#include <set>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/b200.h"
#include "compile.hpp"
#include "driver.hpp"

struct Pool {
  CUdeviceptr ptr = 0;
  size_t bytes = 0;
  // last upload into this pool on the upload stream, and whether `stream` still has to wait for it
  CUevent upload_ev = nullptr;
  bool upload_pending = false;
};

// One GPU: primary context, one non-blocking stream, the (pool id -> slab) table of
// `Slab_alloc` (arrayjit/lib/backend_intf.ml:22-37).
struct b200_dev {
  int ordinal = 0;
  CUdevice dev = 0;
  CUcontext ctx = nullptr;
  CUstream stream = nullptr;
  std::string name;
  int sm_count = 0, cc_major = 0, cc_minor = 0;
  std::mutex mu;
  std::map<int, Pool> pools;
  size_t used = 0;
  volatile unsigned int* status_host = nullptr;  // written by kernels whose bounded waits expire
  CUdeviceptr status_dev = 0;
  // bumped whenever pool 0 (the merge buffer) gets a new slab: a captured graph that reads the
  // merge buffer holds its address and must be captured again
  unsigned long long merge_epoch = 0;
  std::vector<b200_comm*> comms;   // communicators of this device (polled by b200_await when they carry a timeout)
  long long n_launches = 0, n_graph_launches = 0, n_h2d = 0, n_d2h = 0, n_d2d = 0, n_events = 0;

  // Optional second stream for host-to-device copies (b200_set_async_uploads).  A copy waits for
  // the work queued on `stream` before it.  Work queued on `stream` after it waits for the copy if
  // it may touch the copied pool: a routine launch waits for the copies into the pools it binds,
  // every other call for all copies.  A caller that uploads batch i + 1 into a second pool before
  // launching step i therefore overlaps the two, and no hazard the single stream ordered is lost.
  CUstream upload_stream = nullptr;
  CUevent ev_compute = nullptr;
  bool uploads_pending = false;

  void join_pool(Pool& p) {
    if (!p.upload_pending) return;
    p.upload_pending = false;
    b200::cu_check(b200::cu().cuStreamWaitEvent_(stream, p.upload_ev, 0), "cuStreamWaitEvent(upload)");
  }
  void join_pool_id(int pool_id) {
    auto it = pools.find(pool_id);
    if (it != pools.end()) join_pool(it->second);
  }
  void join_all() {
    if (!uploads_pending) return;
    uploads_pending = false;
    for (auto& kv : pools) join_pool(kv.second);
  }
  // `join` = false for the upload itself and for routine launches (which join their own pools)
  void make_current(bool join = true) {
    b200::cu_check(b200::cu().cuCtxSetCurrent_(ctx), "cuCtxSetCurrent");
    if (join) join_all();
  }
  CUdeviceptr address(int pool_id, size_t offset, size_t bytes);
  void check_status();
};

// One NCCL communicator rank (one per process and device) with the stream its collectives run on
// when they overlap a routine.
struct b200_comm {
  b200_dev* dev = nullptr;
  ncclComm_t comm = nullptr;
  int n_ranks = 0, rank = 0;
  CUstream stream = nullptr;     // collectives attached to a routine run here, beside the compute stream
  std::set<struct b200_routine*> routines;   // routines whose runs carry collectives of this communicator
  long long timeout_ms = 0;      // >0: b200_await polls for asynchronous NCCL errors and gives up after this long
  bool aborted = false;
};

// A range of gradients reduced across the ranks as soon as the routine's last stage that writes
// into it has been queued (b200_routine_overlap_allreduce).
struct OverlapBucket {
  int pool_id = 0;
  size_t offset = 0, count = 0;
  int dtype = 0, op = 0;
  int after_stage = -1;          // index of the last stage writing into the range
  CUevent ready = nullptr, done = nullptr;
};

struct b200_event {
  b200_dev* dev = nullptr;
  CUevent ev = nullptr;
};

struct b200_code {
  b200::Code code;
  const std::string* cubin = nullptr;              // generic kernels of the routine
  std::vector<const std::string*> gemm_cubins;     // per stage (null for non-contraction stages)
  // what the code was compiled from, and re-compilations of it in which some top-level statements
  // avoid the forms with alignment demands (made at link when the bound addresses call for it)
  std::string name, ir_text;
  b200::CompileOptions opt;
  std::mutex mu;
  std::map<std::pair<std::set<int>, std::set<int>>, std::unique_ptr<b200_code>> variants;
  b200_code* variant(const std::set<int>& no_pairs_at, const std::set<int>& no_gemm_at);
};

// Parses, plans and compiles a routine to sm_100a machine code (api.cpp).
std::unique_ptr<b200_code> build_code(const std::string& name, const std::string& ir_text, const b200::CompileOptions& opt);

struct GemmLaunch;  // gemm_launch.cpp
struct AttnLaunch;  // gemm_launch.cpp

struct b200_routine {
  b200_dev* dev = nullptr;
  b200_code* code = nullptr;
  CUmodule module = nullptr;
  std::vector<CUmodule> gemm_modules;
  std::vector<CUfunction> fns;                     // per stage
  std::vector<std::vector<CUdeviceptr>> arg_values;  // per stage, one per KArg
  std::vector<GemmLaunch*> gemm;                   // per stage
  std::vector<AttnLaunch*> attn;                   // per stage (fused attention stages)
  std::map<int, CUdeviceptr> node_ptr;
  CUdeviceptr scratch = 0;                         // routine-local nodes
  size_t scratch_bytes = 0;
  std::vector<std::pair<size_t, size_t>> scratch_zero;  // (offset, bytes) cleared every run
  CUdeviceptr statics_dev = 0;
  unsigned int* statics_ring = nullptr;            // page-locked staging
  size_t ring_pos = 0;
  std::vector<long long> last_statics;
  bool statics_valid = false;
  bool want_graph = false;
  bool profiling = false;
  std::vector<std::vector<std::pair<CUevent, CUevent>>> stage_events;  // per stage, per profiled run
  CUgraphExec graph = nullptr;
  bool reads_merge = false;               // some stage takes the merge buffer as an argument
  unsigned long long graph_merge_epoch = 0;  // the device's merge_epoch when `graph` was captured

  b200_comm* overlap_comm = nullptr;
  std::vector<OverlapBucket> buckets;
  bool overlap_warm = false;      // the attached collectives have run once outside a capture
  void enqueue_bucket(OverlapBucket& b);
  std::set<int> pools_used;   // pools of the bound nodes (what a launch has to wait for, uploads-wise)
  b200_code* requested = nullptr;  // the code `link` was given; `code` may be a variant of it
  void link(b200_dev* d, b200_code* c, const b200_binding* b, int n);
  void launch(const int64_t* static_idx, int n_static);
  void enqueue_stages();
  void set_graph(bool on);
  void stage_time(int stage, float* total_ms, int* runs);
  void destroy();
};

// Contraction stages (gemm_launch.cpp)
GemmLaunch* gemm_prepare(b200_routine* r, int stage_index);
void gemm_enqueue(b200_routine* r, int stage_index);
void gemm_release(GemmLaunch* g);
// Fused attention stages (gemm_launch.cpp)
AttnLaunch* attn_prepare(b200_routine* r, int stage_index);
void attn_enqueue(b200_routine* r, int stage_index);
void attn_release(AttnLaunch* a);

// One kernel launch on the device's stream, marked for programmatic stream serialisation
// (runtime.cpp).
void launch_kernel(b200_dev* dev, CUfunction fn, unsigned grid, unsigned bx, unsigned by, unsigned smem, void** args,
                   const char* what, unsigned cluster = 1);
