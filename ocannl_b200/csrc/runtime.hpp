// Run-time objects behind the C ABI: devices with their pool tables and stream, events,
// compiled code and linked routines.
#pragma once
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/b200.h"
#include "compile.hpp"
#include "driver.hpp"

struct Pool {
  CUdeviceptr ptr = 0;
  size_t bytes = 0;
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
  long long n_launches = 0, n_graph_launches = 0, n_h2d = 0, n_d2h = 0, n_d2d = 0, n_events = 0;

  // Optional second stream for host-to-device copies (b200_set_async_uploads).  A copy waits for
  // the work queued on `stream` before it and everything queued on `stream` after it waits for the
  // copy, so every hazard the single stream would have ordered stays ordered -- but a copy no
  // longer waits for the kernels launched AFTER it was queued, nor they for it: a caller that
  // uploads batch i + 1 into a second buffer before launching step i overlaps the two.
  CUstream upload_stream = nullptr;
  CUevent ev_compute = nullptr, ev_upload = nullptr;
  bool uploads_pending = false;

  // `join` = false only for the upload itself: queueing a copy must not make the stream wait for
  // the copies before it (they are ordered among themselves on their own stream)
  void make_current(bool join = true) {
    b200::cu_check(b200::cu().cuCtxSetCurrent_(ctx), "cuCtxSetCurrent");
    if (join && uploads_pending) {
      uploads_pending = false;
      b200::cu_check(b200::cu().cuStreamWaitEvent_(stream, ev_upload, 0), "cuStreamWaitEvent(upload)");
    }
  }
  CUdeviceptr address(int pool_id, size_t offset, size_t bytes);
  void check_status();
};

struct b200_event {
  b200_dev* dev = nullptr;
  CUevent ev = nullptr;
};

struct b200_code {
  b200::Code code;
  const std::string* cubin = nullptr;              // generic kernels of the routine
  std::vector<const std::string*> gemm_cubins;     // per stage (null for non-contraction stages)
};

struct GemmLaunch;  // gemm_launch.cpp

struct b200_routine {
  b200_dev* dev = nullptr;
  b200_code* code = nullptr;
  CUmodule module = nullptr;
  std::vector<CUmodule> gemm_modules;
  std::vector<CUfunction> fns;                     // per stage
  std::vector<std::vector<CUdeviceptr>> arg_values;  // per stage, one per KArg
  std::vector<GemmLaunch*> gemm;                   // per stage
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

// One kernel launch on the device's stream, marked for programmatic stream serialisation
// (runtime.cpp).
void launch_kernel(b200_dev* dev, CUfunction fn, unsigned grid, unsigned bx, unsigned by, unsigned smem, void** args,
                   const char* what, unsigned cluster = 1);
