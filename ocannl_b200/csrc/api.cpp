// C ABI of the backend (include/b200.h): devices, pools, copies, events, routines.
#include "../../include/b200.h"

#include <algorithm>
#include <chrono>
#include <cstring>
#include <map>
#include <thread>
#include <memory>
#include <mutex>
#include <sstream>
#include <vector>

#include "compile.hpp"
#include "driver.hpp"
#include "runtime.hpp"

using namespace b200;

// thread-local message of the last failure; other translation units of the library set it too
thread_local std::string b200_error_slot;
#define g_last_error b200_error_slot

const char* b200_last_error(void) { return g_last_error.c_str(); }
const char* b200_version(void) { return "b200-arrayjit 0.1 (sm_100a)"; }

namespace {

template <class F>
int guard(F&& f) {
  try {
    f();
    return 0;
  } catch (const Error& e) {
    g_last_error = e.what();
    return e.code;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return B200_E_INVALID;
  }
}

void need_driver() {
  if (!cu().loaded) throw Error(B200_E_NO_DEVICE, "the CUDA driver is not available: " + cu().why);
}

std::mutex g_mu;
bool g_inited = false;
std::map<int, std::unique_ptr<b200_dev>> g_devs;

void copy_out(const std::string& s, char* buf, size_t cap) {
  if (!buf || cap == 0) throw Error(B200_E_INVALID, "null output buffer");
  size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
  memcpy(buf, s.data(), n);
  buf[n] = 0;
}

}  // namespace

// ------------------------------------------------------------------ devices
int b200_init(void) {
  return guard([] {
    need_driver();
    std::lock_guard<std::mutex> g(g_mu);
    if (g_inited) return;
    cu_check(cu().cuInit_(0), "cuInit");
    g_inited = true;
  });
}

int b200_num_devices(int* out) {
  return guard([&] {
    if (!out) throw Error(B200_E_INVALID, "null argument");
    int rc = b200_init();
    if (rc) throw Error(rc, g_last_error);
    cu_check(cu().cuDeviceGetCount_(out), "cuDeviceGetCount");
  });
}

int b200_device_open(int ordinal, b200_dev** out) {
  return guard([&] {
    if (!out) throw Error(B200_E_INVALID, "null argument");
    int n = 0;
    int rc = b200_num_devices(&n);
    if (rc) throw Error(rc, g_last_error);
    if (ordinal < 0 || ordinal >= n) throw Error(B200_E_INVALID, "device ordinal out of range");
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_devs.find(ordinal);
    if (it != g_devs.end()) {
      *out = it->second.get();
      return;
    }
    auto d = std::make_unique<b200_dev>();
    d->ordinal = ordinal;
    cu_check(cu().cuDeviceGet_(&d->dev, ordinal), "cuDeviceGet");
    cu_check(cu().cuDevicePrimaryCtxRetain_(&d->ctx, d->dev), "cuDevicePrimaryCtxRetain");
    d->make_current();
    cu_check(cu().cuStreamCreate_(&d->stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate");
    char name[128] = {0};
    cu().cuDeviceGetName_(name, sizeof name, d->dev);
    d->name = name;
    cu().cuDeviceGetAttribute_(&d->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, d->dev);
    cu().cuDeviceGetAttribute_(&d->cc_major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, d->dev);
    cu().cuDeviceGetAttribute_(&d->cc_minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, d->dev);
    // device-side status word, written by kernels whose bounded waits expire
    void* hp = nullptr;
    cu_check(cu().cuMemHostAlloc_(&hp, 256, CU_MEMHOSTALLOC_DEVICEMAP | CU_MEMHOSTALLOC_PORTABLE), "cuMemHostAlloc");
    d->status_host = (volatile unsigned int*)hp;   // words 0-1: status, 2-31: developer trace
    memset(hp, 0, 256);
    cu_check(cu().cuMemHostGetDevicePointer_(&d->status_dev, hp, 0), "cuMemHostGetDevicePointer");
    *out = d.get();
    g_devs[ordinal] = std::move(d);
  });
}

int b200_device_props(b200_dev* dev, char* json, size_t cap) {
  return guard([&] {
    if (!dev) throw Error(B200_E_INVALID, "null device");
    std::ostringstream o;
    size_t total = 0;
    cu().cuDeviceTotalMem_(&total, dev->dev);
    o << "{\"ordinal\":" << dev->ordinal << ",\"name\":\"" << dev->name << "\",\"sm_count\":" << dev->sm_count
      << ",\"compute_capability\":\"" << dev->cc_major << "." << dev->cc_minor << "\",\"total_memory\":" << total << "}";
    copy_out(o.str(), json, cap);
  });
}

// -------------------------------------------------------------------- pools
int b200_pool_alloc(b200_dev* dev, int pool_id, size_t bytes, size_t alignment) {
  return guard([&] {
    if (!dev || pool_id < 0) throw Error(B200_E_INVALID, "bad pool arguments");
    (void)alignment;  // cuMemAlloc returns 256-byte aligned memory, above any element size
    dev->make_current();
    std::lock_guard<std::mutex> g(dev->mu);
    auto it = dev->pools.find(pool_id);
    if (it != dev->pools.end()) {
      cu_check(cu().cuStreamSynchronize_(dev->stream), "cuStreamSynchronize");
      cu_check(cu().cuMemFree_(it->second.ptr), "cuMemFree");
      if (it->second.upload_ev) cu().cuEventDestroy_(it->second.upload_ev);
      dev->used -= it->second.bytes;
      dev->pools.erase(it);
    }
    Pool p;
    p.bytes = bytes;
    if (pool_id == 0) dev->merge_epoch++;
    cu_check(cu().cuMemAlloc_(&p.ptr, bytes ? bytes : 1), "cuMemAlloc");
    dev->used += bytes;
    dev->pools[pool_id] = p;
  });
}

int b200_pool_free(b200_dev* dev, int pool_id) {
  return guard([&] {
    if (!dev) throw Error(B200_E_INVALID, "null device");
    dev->make_current();
    std::lock_guard<std::mutex> g(dev->mu);
    auto it = dev->pools.find(pool_id);
    if (it == dev->pools.end()) throw Error(B200_E_INVALID, "free_pool: unknown pool id " + std::to_string(pool_id));
    if (pool_id == 0) dev->merge_epoch++;
    cu_check(cu().cuStreamSynchronize_(dev->stream), "cuStreamSynchronize");
    cu_check(cu().cuMemFree_(it->second.ptr), "cuMemFree");
    if (it->second.upload_ev) cu().cuEventDestroy_(it->second.upload_ev);
    dev->used -= it->second.bytes;
    dev->pools.erase(it);
  });
}

int b200_pool_memset0(b200_dev* dev, int pool_id, size_t offset, size_t bytes) {
  return guard([&] {
    if (!dev) throw Error(B200_E_INVALID, "null device");
    dev->make_current(/*join=*/false);
    dev->join_pool_id(pool_id);   // only uploads into this pool matter to the clear
    CUdeviceptr p = dev->address(pool_id, offset, bytes);
    if (bytes) cu_check(cu().cuMemsetD8Async_(p, 0, bytes, dev->stream), "cuMemsetD8Async");
  });
}

int b200_pool_address(b200_dev* dev, int pool_id, uint64_t* device_ptr, size_t* bytes) {
  return guard([&] {
    if (!dev) throw Error(B200_E_INVALID, "null device");
    std::lock_guard<std::mutex> g(dev->mu);
    auto it = dev->pools.find(pool_id);
    if (it == dev->pools.end()) throw Error(B200_E_INVALID, "unknown pool id " + std::to_string(pool_id));
    if (device_ptr) *device_ptr = (uint64_t)it->second.ptr;
    if (bytes) *bytes = it->second.bytes;
  });
}

// ------------------------------------------------------------------- copies
int b200_h2d(b200_dev* dev, int pool_id, size_t offset, const void* src, size_t bytes) {
  return guard([&] {
    if (!dev || (!src && bytes)) throw Error(B200_E_INVALID, "null argument");
    dev->make_current(/*join=*/dev->upload_stream == nullptr);
    CUdeviceptr p = dev->address(pool_id, offset, bytes);
    if (bytes && dev->upload_stream) {
      Pool& pool = dev->pools.at(pool_id);
      if (!pool.upload_ev) cu_check(cu().cuEventCreate_(&pool.upload_ev, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
      cu_check(cu().cuEventRecord_(dev->ev_compute, dev->stream), "cuEventRecord");
      cu_check(cu().cuStreamWaitEvent_(dev->upload_stream, dev->ev_compute, 0), "cuStreamWaitEvent");
      cu_check(cu().cuMemcpyHtoDAsync_(p, src, bytes, dev->upload_stream), "cuMemcpyHtoDAsync");
      cu_check(cu().cuEventRecord_(pool.upload_ev, dev->upload_stream), "cuEventRecord");
      pool.upload_pending = true;
      dev->uploads_pending = true;
    } else if (bytes) {
      cu_check(cu().cuMemcpyHtoDAsync_(p, src, bytes, dev->stream), "cuMemcpyHtoDAsync");
    }
    dev->n_h2d++;
  });
}

int b200_d2h(b200_dev* dev, int pool_id, size_t offset, void* dst, size_t bytes) {
  return guard([&] {
    if (!dev || (!dst && bytes)) throw Error(B200_E_INVALID, "null argument");
    dev->make_current(/*join=*/false);
    dev->join_pool_id(pool_id);
    CUdeviceptr p = dev->address(pool_id, offset, bytes);
    if (bytes) cu_check(cu().cuMemcpyDtoHAsync_(dst, p, bytes, dev->stream), "cuMemcpyDtoHAsync");
    dev->n_d2h++;
  });
}

static void d2d_raw(b200_dev* dst_dev, CUdeviceptr dst, b200_dev* src_dev, CUdeviceptr src, size_t bytes) {
  if (!bytes) return;
  dst_dev->make_current();
  if (dst_dev == src_dev) {
    cu_check(cu().cuMemcpyDtoDAsync_(dst, src, bytes, dst_dev->stream), "cuMemcpyDtoDAsync");
  } else {
    // order after everything queued on the source stream, then copy on the destination stream
    CUevent ev;
    src_dev->make_current();
    cu_check(cu().cuEventCreate_(&ev, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
    cu_check(cu().cuEventRecord_(ev, src_dev->stream), "cuEventRecord");
    dst_dev->make_current();
    cu_check(cu().cuStreamWaitEvent_(dst_dev->stream, ev, 0), "cuStreamWaitEvent");
    cu_check(cu().cuMemcpyPeerAsync_(dst, dst_dev->ctx, src, src_dev->ctx, bytes, dst_dev->stream), "cuMemcpyPeerAsync");
    cu().cuEventDestroy_(ev);
  }
  dst_dev->n_d2d++;
}

int b200_d2d(b200_dev* dst_dev, int dst_pool, size_t dst_offset, b200_dev* src_dev, int src_pool, size_t src_offset,
             size_t bytes) {
  return guard([&] {
    if (!dst_dev || !src_dev) throw Error(B200_E_INVALID, "null device");
    d2d_raw(dst_dev, dst_dev->address(dst_pool, dst_offset, bytes), src_dev, src_dev->address(src_pool, src_offset, bytes),
            bytes);
  });
}

int b200_merge_copy(b200_dev* dst_dev, b200_dev* src_dev, int src_pool, size_t src_offset, size_t bytes) {
  return guard([&] {
    if (!dst_dev || !src_dev) throw Error(B200_E_INVALID, "null device");
    size_t have = 0;
    {
      std::lock_guard<std::mutex> g(dst_dev->mu);
      auto it = dst_dev->pools.find(0);
      if (it != dst_dev->pools.end()) have = it->second.bytes;
    }
    if (have < bytes) {
      // grow geometrically, like the cuda backend's merge buffer (arrayjit/lib/cuda_backend.ml:130-134)
      size_t want = bytes + bytes / 5;
      int rc = b200_pool_alloc(dst_dev, 0, want, 256);
      if (rc) throw Error(rc, g_last_error);
    }
    d2d_raw(dst_dev, dst_dev->address(0, 0, bytes), src_dev, src_dev->address(src_pool, src_offset, bytes), bytes);
  });
}

int b200_host_alloc(size_t bytes, void** out) {
  return guard([&] {
    need_driver();
    if (!out) throw Error(B200_E_INVALID, "null argument");
    if (g_devs.empty()) throw Error(B200_E_INVALID, "open a device before allocating page-locked memory");
    g_devs.begin()->second->make_current();
    cu_check(cu().cuMemHostAlloc_(out, bytes ? bytes : 1, CU_MEMHOSTALLOC_PORTABLE), "cuMemHostAlloc");
  });
}

int b200_host_free(void* p) {
  return guard([&] {
    need_driver();
    if (p) cu_check(cu().cuMemFreeHost_(p), "cuMemFreeHost");
  });
}

// ------------------------------------------------------------------- events
static void await_polling(b200_dev* dev, CUevent until);
int b200_event_record(b200_dev* dev, b200_event** out) {
  return guard([&] {
    if (!dev || !out) throw Error(B200_E_INVALID, "null argument");
    dev->make_current();
    auto* e = new b200_event();
    e->dev = dev;
    cu_check(cu().cuEventCreate_(&e->ev, CU_EVENT_DEFAULT), "cuEventCreate");
    cu_check(cu().cuEventRecord_(e->ev, dev->stream), "cuEventRecord");
    dev->n_events++;
    *out = e;
  });
}

int b200_event_query(b200_event* ev, int* done) {
  return guard([&] {
    if (!ev || !done) throw Error(B200_E_INVALID, "null argument");
    CUresult r = cu().cuEventQuery_(ev->ev);
    if (r == CUDA_SUCCESS) *done = 1;
    else if (r == CUDA_ERROR_NOT_READY) *done = 0;
    else cu_check(r, "cuEventQuery");
  });
}

int b200_event_sync(b200_event* ev) {
  return guard([&] {
    if (!ev) throw Error(B200_E_INVALID, "null argument");
    ev->dev->make_current();
    await_polling(ev->dev, ev->ev);    // polls like b200_await when a communicator carries a timeout
    ev->dev->check_status();
  });
}

int b200_event_elapsed_ms(b200_event* start, b200_event* stop, float* ms) {
  return guard([&] {
    if (!start || !stop || !ms) throw Error(B200_E_INVALID, "null argument");
    cu_check(cu().cuEventElapsedTime_(ms, start->ev, stop->ev), "cuEventElapsedTime");
  });
}

int b200_event_free(b200_event* ev) {
  return guard([&] {
    if (!ev) return;
    cu().cuEventDestroy_(ev->ev);
    delete ev;
  });
}

int b200_stream_wait(b200_dev* dev, b200_event* ev) {
  return guard([&] {
    if (!dev || !ev) throw Error(B200_E_INVALID, "null argument");
    dev->make_current();
    cu_check(cu().cuStreamWaitEvent_(dev->stream, ev->ev, 0), "cuStreamWaitEvent");
  });
}

// Waits for the device's stream.  When a communicator of the device carries a timeout, the wait
// is a poll: NCCL reports a failed peer or a broken link asynchronously
// (ncclCommGetAsyncError), and a collective whose peer never arrives would otherwise keep the
// stream, and this call, busy for ever.  On an asynchronous error, or when the timeout passes
// with the stream still busy, the communicator is aborted (ncclCommAbort ends its kernels) and
// the error is returned; the device stays usable.
static void await_polling(b200_dev* dev, CUevent until) {
  auto block = [&] {
    if (until) cu_check(cu().cuEventSynchronize_(until), "cuEventSynchronize");
    else cu_check(cu().cuStreamSynchronize_(dev->stream), "cuStreamSynchronize");
  };
  long long limit = 0;
  for (auto* c : dev->comms)
    if (c->timeout_ms > 0 && !c->aborted) limit = limit ? std::min(limit, c->timeout_ms) : c->timeout_ms;
  if (!limit) {
    block();
    return;
  }
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    CUresult q = until ? cu().cuEventQuery_(until) : cu().cuStreamQuery_(dev->stream);
    if (q == CUDA_SUCCESS) return;
    if (q != CUDA_ERROR_NOT_READY) cu_check(q, "cuStreamQuery");
    const long long waited = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    for (auto* c : dev->comms) {
      if (c->aborted || c->timeout_ms <= 0) continue;
      ncclResult_t async = ncclSuccess;
      ncclResult_t r = nccl().ncclCommGetAsyncError_(c->comm, &async);
      const bool failed = r != ncclSuccess || (async != ncclSuccess && async != ncclInProgress);
      if (failed || waited > c->timeout_ms) {
        nccl().ncclCommAbort_(c->comm);
        c->aborted = true;
        cu().cuStreamSynchronize_(dev->stream);   // the aborted collective's kernels end
        if (failed)
          throw Error(r != ncclSuccess ? (int)r : (int)async, std::string("NCCL reported an asynchronous error: ") +
                                                                    nccl().ncclGetErrorString_(r != ncclSuccess ? r : async) +
                                                                    "; the communicator was aborted");
        throw Error(B200_E_DEVICE, "a collective did not finish within " + std::to_string(c->timeout_ms) +
                                       " ms (is a rank missing?); the communicator was aborted");
      }
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}

int b200_await(b200_dev* dev) {
  return guard([&] {
    if (!dev) throw Error(B200_E_INVALID, "null device");
    dev->make_current();
    await_polling(dev, nullptr);
    dev->check_status();
  });
}

int b200_is_idle(b200_dev* dev, int* idle) {
  return guard([&] {
    if (!dev || !idle) throw Error(B200_E_INVALID, "null argument");
    CUresult r = cu().cuStreamQuery_(dev->stream);
    if (r == CUDA_SUCCESS) *idle = 1;
    else if (r == CUDA_ERROR_NOT_READY) *idle = 0;
    else cu_check(r, "cuStreamQuery");
  });
}

int b200_set_async_uploads(b200_dev* dev, int on) {
  return guard([&] {
    if (!dev) throw Error(B200_E_INVALID, "null argument");
    dev->make_current();
    if (on && !dev->upload_stream) {
      cu_check(cu().cuStreamCreate_(&dev->upload_stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate");
      cu_check(cu().cuEventCreate_(&dev->ev_compute, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
    } else if (!on && dev->upload_stream) {
      cu_check(cu().cuStreamSynchronize_(dev->upload_stream), "cuStreamSynchronize");
      cu().cuStreamDestroy_(dev->upload_stream);
      cu().cuEventDestroy_(dev->ev_compute);
      for (auto& kv : dev->pools) {
        if (kv.second.upload_ev) cu().cuEventDestroy_(kv.second.upload_ev);
        kv.second.upload_ev = nullptr;
        kv.second.upload_pending = false;
      }
      dev->upload_stream = nullptr;
      dev->ev_compute = nullptr;
      dev->uploads_pending = false;
    }
  });
}

int b200_stream_handle(b200_dev* dev, uint64_t* custream) {
  return guard([&] {
    if (!dev || !custream) throw Error(B200_E_INVALID, "null argument");
    *custream = (uint64_t)dev->stream;
  });
}

// ----------------------------------------------------------------- routines
int b200_compile(const char* name, const char* ir, size_t len, const char* options, b200_code** out) {
  return guard([&] {
    if (!ir || !out) throw Error(B200_E_INVALID, "null argument");
    CompileOptions opt;
    if (options) {
      std::istringstream is(options);
      std::string kv;
      while (is >> kv) {
        size_t eq = kv.find('=');
        std::string k = kv.substr(0, eq), v = eq == std::string::npos ? "1" : kv.substr(eq + 1);
        bool on = v != "0";
        if (k == "gemm") opt.enable_gemm = on;
        else if (k == "attn") opt.enable_attn = on;
        else if (k == "coop") opt.enable_coop = on;
        else if (k == "fuse") opt.enable_fuse = on;
        else if (k == "pairs") opt.enable_pairs = on;
        else if (k == "splitk") opt.enable_splitk = on;
        else if (k == "tf32") opt.enable_tf32 = on;
        else if (k == "large_models") opt.large_models = on;
        else if (k == "bounds") opt.bounds = on;
        else throw Error(B200_E_INVALID, "unknown compile option '" + k + "'");
      }
    }
    if (opt.bounds) opt.enable_gemm = opt.enable_attn = opt.enable_pairs = false;   // the checked accesses are the generic kernels'
    *out = build_code(name ? name : "", std::string(ir, len), opt).release();
  });
}

std::unique_ptr<b200_code> build_code(const std::string& name, const std::string& ir_text, const CompileOptions& opt) {
  Program p = parse_program(ir_text.data(), ir_text.size());
  if (!name.empty()) p.name = name;
  auto code = std::make_unique<b200_code>();
  code->name = name;
  code->ir_text = ir_text;
  code->opt = opt;
  code->code = compile_program(std::move(p), opt);
  // machine code for sm_100a is produced here, device independent
  bool any_generic = false;
  for (auto& s : code->code.stages) any_generic |= s.kind == Stage::Generic;
  if (any_generic) code->cubin = &compile_cubin(code->code.source, code->code.prog.name);
  for (auto& s : code->code.stages)
    if (s.own_module()) code->gemm_cubins.push_back(&compile_cubin(s.gemm_source, s.kernel));
    else code->gemm_cubins.push_back(nullptr);
  return code;
}

b200_code* b200_code::variant(const std::set<int>& no_pairs_at, const std::set<int>& no_gemm_at) {
  std::lock_guard<std::mutex> g(mu);
  auto key = std::make_pair(no_pairs_at, no_gemm_at);
  auto it = variants.find(key);
  if (it != variants.end()) return it->second.get();
  CompileOptions o = opt;
  o.no_pairs_at = no_pairs_at;
  o.no_gemm_at = no_gemm_at;
  auto v = build_code(name, ir_text, o);
  b200_code* raw = v.get();
  variants[key] = std::move(v);
  return raw;
}

int b200_routine_info(b200_routine* r, char* json, size_t cap) {
  return guard([&] {
    if (!r) throw Error(B200_E_INVALID, "null routine");
    copy_out(r->code->code.describe(), json, cap);
  });
}

int b200_code_info(b200_code* code, char* json, size_t cap) {
  return guard([&] {
    if (!code) throw Error(B200_E_INVALID, "null code");
    copy_out(code->code.describe(), json, cap);
  });
}

int b200_code_source(b200_code* code, int stage, char* buf, size_t cap, size_t* needed) {
  return guard([&] {
    if (!code) throw Error(B200_E_INVALID, "null code");
    const std::string* s = &code->code.source;
    if (stage >= 0) {
      if (stage >= (int)code->code.stages.size()) throw Error(B200_E_INVALID, "stage out of range");
      if (code->code.stages[stage].own_module()) s = &code->code.stages[stage].gemm_source;
    }
    if (needed) *needed = s->size() + 1;
    if (buf && cap) copy_out(*s, buf, cap);
  });
}

int b200_code_free(b200_code* code) {
  return guard([&] { delete code; });
}

int b200_link(b200_dev* dev, b200_code* code, const b200_binding* bindings, int n, b200_routine** out) {
  return guard([&] {
    if (!dev || !code || !out || (n > 0 && !bindings)) throw Error(B200_E_INVALID, "null argument");
    dev->make_current();
    auto r = std::make_unique<b200_routine>();
    r->link(dev, code, bindings, n);
    *out = r.release();
  });
}

int b200_launch(b200_routine* r, const int64_t* static_idx, int n_static) {
  return guard([&] {
    if (!r) throw Error(B200_E_INVALID, "null routine");
    r->dev->make_current(/*join=*/false);
    if (r->dev->uploads_pending) {
      r->dev->join_pool_id(0);   // the merge buffer
      for (int id : r->pools_used) r->dev->join_pool_id(id);
    }
    r->launch(static_idx, n_static);
  });
}

int b200_routine_use_graph(b200_routine* r, int enable) {
  return guard([&] {
    if (!r) throw Error(B200_E_INVALID, "null routine");
    r->set_graph(enable != 0);
  });
}

int b200_routine_launch_count(b200_routine* r, int64_t* kernels_per_run) {
  return guard([&] {
    if (!r || !kernels_per_run) throw Error(B200_E_INVALID, "null argument");
    int64_t k = 0;
    for (auto& s : r->code->code.stages) k += s.kind != Stage::Memset;
    *kernels_per_run = k;
  });
}

int b200_routine_profile(b200_routine* r, int enable) {
  return guard([&] {
    if (!r) throw Error(B200_E_INVALID, "null routine");
    r->profiling = enable != 0;
  });
}

int b200_routine_stage_time(b200_routine* r, int stage, float* total_ms, int* runs) {
  return guard([&] {
    if (!r || !total_ms || !runs) throw Error(B200_E_INVALID, "null argument");
    r->dev->make_current();
    r->stage_time(stage, total_ms, runs);
  });
}

int b200_routine_free(b200_routine* r) {
  return guard([&] {
    if (!r) return;
    r->dev->make_current();
    r->destroy();
    delete r;
  });
}

// ------------------------------------------------------------ observability
int b200_used_memory(b200_dev* dev, size_t* bytes) {
  return guard([&] {
    if (!dev || !bytes) throw Error(B200_E_INVALID, "null argument");
    *bytes = dev->used;
  });
}

int b200_debug_info(b200_dev* dev, char* json, size_t cap) {
  return guard([&] {
    if (!dev) throw Error(B200_E_INVALID, "null device");
    std::ostringstream o;
    o << "{\"pools\":" << dev->pools.size() << ",\"used_bytes\":" << dev->used << ",\"kernel_launches\":" << dev->n_launches
      << ",\"graph_launches\":" << dev->n_graph_launches << ",\"h2d\":" << dev->n_h2d << ",\"d2h\":" << dev->n_d2h
      << ",\"d2d\":" << dev->n_d2d << ",\"events\":" << dev->n_events << "}";
    copy_out(o.str(), json, cap);
  });
}

// ------------------------------------------------------------- data parallel
static void nccl_check(ncclResult_t r, const char* what) {
  if (r == ncclSuccess) return;
  throw Error((int)r, std::string(what) + ": " + nccl().ncclGetErrorString_(r));
}

int b200_comm_unique_id(char* id128) {
  return guard([&] {
    if (!id128) throw Error(B200_E_INVALID, "null argument");
    if (!nccl().loaded) throw Error(B200_E_NO_DEVICE, "NCCL is not available: " + nccl().why);
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    ncclUniqueId id;
    nccl_check(nccl().ncclGetUniqueId_(&id), "ncclGetUniqueId");
    memcpy(id128, &id, 128);
  });
}

int b200_comm_init_rank(b200_dev* dev, int n_ranks, int rank, const char* id128, b200_comm** out) {
  return guard([&] {
    if (!dev || !id128 || !out) throw Error(B200_E_INVALID, "null argument");
    if (n_ranks < 1 || rank < 0 || rank >= n_ranks) throw Error(B200_E_INVALID, "bad rank / world size");
    if (!nccl().loaded) throw Error(B200_E_NO_DEVICE, "NCCL is not available: " + nccl().why);
    dev->make_current();
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    auto c = std::make_unique<b200_comm>();
    c->dev = dev;
    c->n_ranks = n_ranks;
    c->rank = rank;
    nccl_check(nccl().ncclCommInitRank_(&c->comm, n_ranks, id, rank), "ncclCommInitRank");
    cu_check(cu().cuStreamCreate_(&c->stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate(communicator)");
    dev->comms.push_back(c.get());
    *out = c.release();
  });
}

// One process driving all shards (the reference's arrangement: lib/parallel.ml:166-208 keeps every
// shard's context in one process): the communicators of n devices at once, and an allreduce over
// one range per device issued as one NCCL group -- a single thread that manages several devices
// must group its calls, or the first one would wait for ranks that the same thread has yet to call.
int b200_comm_init_all(int n, b200_dev* const* devs, b200_comm** out) {
  return guard([&] {
    if (n < 1 || !devs || !out) throw Error(B200_E_INVALID, "bad arguments");
    if (!nccl().loaded) throw Error(B200_E_NO_DEVICE, "NCCL is not available: " + nccl().why);
    std::vector<int> ordinals;
    std::vector<ncclComm_t> comms((size_t)n, nullptr);
    for (int i = 0; i < n; ++i) {
      if (!devs[i]) throw Error(B200_E_INVALID, "null device");
      ordinals.push_back(devs[i]->ordinal);
    }
    nccl_check(nccl().ncclCommInitAll_(comms.data(), n, ordinals.data()), "ncclCommInitAll");
    for (int i = 0; i < n; ++i) {
      auto c = std::make_unique<b200_comm>();
      c->dev = devs[i];
      c->n_ranks = n;
      c->rank = i;
      c->comm = comms[(size_t)i];
      devs[i]->make_current();
      cu_check(cu().cuStreamCreate_(&c->stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate(communicator)");
      devs[i]->comms.push_back(c.get());
      out[i] = c.release();
    }
  });
}

int b200_allreduce_all(int n, b200_comm* const* comms, const int* pool_ids, const size_t* offsets, size_t count, int dtype,
                       int op) {
  return guard([&] {
    if (n < 1 || !comms || !pool_ids || !offsets) throw Error(B200_E_INVALID, "bad arguments");
    if (dtype != B200_F32 && dtype != B200_BF16) throw Error(B200_E_INVALID, "bad dtype");
    if (op != B200_SUM && op != B200_AVG) throw Error(B200_E_INVALID, "bad reduction");
    const size_t esz = dtype == B200_F32 ? 4 : 2;
    std::vector<CUdeviceptr> ptrs;
    for (int i = 0; i < n; ++i) {
      if (!comms[i] || comms[i]->aborted) throw Error(B200_E_INVALID, "null or aborted communicator");
      ptrs.push_back(comms[i]->dev->address(pool_ids[i], offsets[i], count * esz));
    }
    nccl_check(nccl().ncclGroupStart_(), "ncclGroupStart");
    ncclResult_t first = ncclSuccess;
    for (int i = 0; i < n; ++i) {
      b200_dev* dev = comms[i]->dev;
      dev->make_current();
      ncclResult_t r = nccl().ncclAllReduce_((const void*)ptrs[(size_t)i], (void*)ptrs[(size_t)i], count,
                                             dtype == B200_F32 ? ncclFloat32 : ncclBfloat16, op == B200_SUM ? ncclSum : ncclAvg,
                                             comms[i]->comm, (cudaStream_t)dev->stream);
      if (r != ncclSuccess && first == ncclSuccess) first = r;
    }
    ncclResult_t e = nccl().ncclGroupEnd_();
    nccl_check(first, "ncclAllReduce(group)");
    nccl_check(e, "ncclGroupEnd");
  });
}

int b200_allreduce(b200_comm* comm, int pool_id, size_t offset, size_t count, int dtype, int op) {
  return guard([&] {
    if (!comm) throw Error(B200_E_INVALID, "null communicator");
    if (dtype != B200_F32 && dtype != B200_BF16) throw Error(B200_E_INVALID, "bad dtype");
    if (op != B200_SUM && op != B200_AVG) throw Error(B200_E_INVALID, "bad reduction");
    if (comm->aborted) throw Error(B200_E_INVALID, "the communicator was aborted");
    b200_dev* dev = comm->dev;
    dev->make_current();
    size_t esz = dtype == B200_F32 ? 4 : 2;
    CUdeviceptr p = dev->address(pool_id, offset, count * esz);
    nccl_check(nccl().ncclAllReduce_((const void*)p, (void*)p, count, dtype == B200_F32 ? ncclFloat32 : ncclBfloat16,
                                     op == B200_SUM ? ncclSum : ncclAvg, comm->comm, (cudaStream_t)dev->stream),
               "ncclAllReduce");
  });
}

int b200_comm_set_timeout(b200_comm* comm, long long timeout_ms) {
  return guard([&] {
    if (!comm) throw Error(B200_E_INVALID, "null communicator");
    comm->timeout_ms = timeout_ms > 0 ? timeout_ms : 0;
  });
}

int b200_routine_overlap_allreduce(b200_routine* r, b200_comm* comm, int n, const int* pool_ids, const size_t* offsets,
                                   const size_t* counts, int dtype, int op) {
  return guard([&] {
    if (!r || (n > 0 && (!comm || !pool_ids || !offsets || !counts))) throw Error(B200_E_INVALID, "null argument");
    if (dtype != B200_F32 && dtype != B200_BF16) throw Error(B200_E_INVALID, "bad dtype");
    if (op != B200_SUM && op != B200_AVG) throw Error(B200_E_INVALID, "bad reduction");
    if (n > 0 && comm->dev != r->dev) throw Error(B200_E_INVALID, "the communicator belongs to another device");
    if (n > 0 && comm->aborted) throw Error(B200_E_INVALID, "the communicator was aborted");
    r->dev->make_current();
    r->set_graph(false);   // a captured graph would not hold the new collectives
    for (auto& b : r->buckets) {
      if (b.ready) cu().cuEventDestroy_(b.ready);
      if (b.done) cu().cuEventDestroy_(b.done);
    }
    r->buckets.clear();
    r->overlap_warm = false;
    if (r->overlap_comm) r->overlap_comm->routines.erase(r);
    r->overlap_comm = n > 0 ? comm : nullptr;
    if (n > 0) comm->routines.insert(r);
    const Program& P = r->code->code.prog;
    const size_t esz = dtype == B200_F32 ? 4 : 2;
    for (int k = 0; k < n; ++k) {
      OverlapBucket b;
      b.pool_id = pool_ids[k];
      b.offset = offsets[k];
      b.count = counts[k];
      b.dtype = dtype;
      b.op = op;
      const CUdeviceptr lo = r->dev->address(b.pool_id, b.offset, b.count * esz), hi = lo + b.count * esz;
      // the last stage that writes a node overlapping the range
      for (size_t i = 0; i < r->code->code.stages.size(); ++i)
        for (int tn : r->code->code.stages[i].writes) {
          auto it = r->node_ptr.find(tn);
          if (it == r->node_ptr.end()) continue;
          const CUdeviceptr a = it->second, e = a + (CUdeviceptr)P.tn(tn).bytes();
          if (a < hi && lo < e) b.after_stage = (int)i;
        }
      cu_check(cu().cuEventCreate_(&b.ready, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
      cu_check(cu().cuEventCreate_(&b.done, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
      r->buckets.push_back(b);
    }
  });
}

int b200_comm_free(b200_comm* comm) {
  return guard([&] {
    if (!comm) return;
    b200_dev* dev = comm->dev;
    // A captured graph that holds collectives of this communicator keeps the communicator in use:
    // NCCL waits for such graphs to be destroyed before it lets the communicator go.  Routines that
    // carry its collectives lose them (and their graphs) here.
    for (b200_routine* r : comm->routines) {
      r->dev->make_current();
      r->set_graph(false);
      for (auto& b : r->buckets) {
        if (b.ready) cu().cuEventDestroy_(b.ready);
        if (b.done) cu().cuEventDestroy_(b.done);
      }
      r->buckets.clear();
      r->overlap_comm = nullptr;
    }
    comm->routines.clear();
    if (dev) {
      dev->make_current();
      for (size_t i = 0; i < dev->comms.size(); ++i)
        if (dev->comms[i] == comm) { dev->comms.erase(dev->comms.begin() + (long)i); break; }
    }
    if (comm->comm && !comm->aborted) nccl().ncclCommDestroy_(comm->comm);
    if (comm->stream) cu().cuStreamDestroy_(comm->stream);
    delete comm;
  });
}
