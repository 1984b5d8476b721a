// dlopen-based bindings to libcuda / libnvrtc / libnccl and the NVRTC compile cache.
#include "driver.hpp"

#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <vector>

namespace b200 {

#define B200_STR2(x) #x
#define B200_STR(x) B200_STR2(x)

// The libraries are opened with RTLD_LOCAL: their symbols must not enter the global namespace, where
// they would shadow those of another copy loaded later (a Python process that imports a framework
// bundling its own, newer NCCL after this library opened the system's would fail to resolve).
static void* open_first(const std::vector<std::string>& names, std::string* why) {
  for (auto& n : names) {
    if (n.empty()) continue;
    void* h = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (h) return h;
    *why += n + ": " + dlerror() + "; ";
  }
  return nullptr;
}

static std::string env(const char* k) {
  const char* v = getenv(k);
  return v ? v : "";
}

CuApi& cu() {
  static CuApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = open_first({env("B200_LIBCUDA"), "libcuda.so.1", "libcuda.so"}, &api.why);
    if (!h) return;
    bool ok = true;
    // the header maps unversioned names to their current ABI (cuMemAlloc -> cuMemAlloc_v2);
    // B200_STR(name) stringises the mapped name
#define X(name)                                                      \
  api.name##_ = (decltype(&::name))dlsym(h, B200_STR(name));         \
  if (!api.name##_) { ok = false; api.why += "missing " B200_STR(name) "; "; }
    B200_CU_FUNCS(X)
#undef X
    api.loaded = ok;
  });
  return api;
}

NvrtcApi& nvrtc() {
  static NvrtcApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = open_first({env("B200_LIBNVRTC"), "libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so"},
                         &api.why);
    if (!h) return;
    bool ok = true;
#define X(name)                                              \
  api.name##_ = (decltype(&::name))dlsym(h, #name);          \
  if (!api.name##_) { ok = false; api.why += "missing " #name "; "; }
    B200_NVRTC_FUNCS(X)
#undef X
    api.loaded = ok;
  });
  return api;
}

NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = open_first({env("B200_LIBNCCL"), "libnccl.so.2", "libnccl.so"}, &api.why);
    if (!h) return;
    bool ok = true;
#define X(name)                                              \
  api.name##_ = (decltype(&::name))dlsym(h, #name);          \
  if (!api.name##_) { ok = false; api.why += "missing " #name "; "; }
    B200_NCCL_FUNCS(X)
#undef X
    api.loaded = ok;
  });
  return api;
}

void cu_check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  const char* msg = nullptr;
  if (cu().loaded) cu().cuGetErrorString_(r, &msg);
  throw Error((int)r, std::string(what) + ": " + (msg ? msg : "CUDA error") + " (CUresult " + std::to_string((int)r) + ")");
}

const std::string& compile_cubin(const std::string& source, const std::string& name, std::string* log_out) {
  static std::mutex mu;
  static std::map<std::string, std::string> cache;
  // the extra flags are part of what is compiled
  const std::string key = source + "\n// flags: " + env("B200_NVRTC_FLAGS");
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  NvrtcApi& n = nvrtc();
  if (!n.loaded) throw Error(-2, "NVRTC is not available: " + n.why);
  nvrtcProgram prog;
  nvrtcResult r = n.nvrtcCreateProgram_(&prog, source.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr);
  if (r != NVRTC_SUCCESS) throw Error((int)r, std::string("nvrtcCreateProgram: ") + n.nvrtcGetErrorString_(r));
  std::vector<const char*> opts = {"--gpu-architecture=sm_100a", "-lineinfo", "--std=c++17", "-default-device"};
  std::string extra = env("B200_NVRTC_FLAGS");
  std::vector<std::string> extra_v;
  for (size_t p = 0; p < extra.size();) {
    size_t q = extra.find(' ', p);
    if (q == std::string::npos) q = extra.size();
    if (q > p) extra_v.push_back(extra.substr(p, q - p));
    p = q + 1;
  }
  for (auto& s : extra_v) opts.push_back(s.c_str());
  r = n.nvrtcCompileProgram_(prog, (int)opts.size(), opts.data());
  std::string log;
  size_t ls = 0;
  if (n.nvrtcGetProgramLogSize_(prog, &ls) == NVRTC_SUCCESS && ls > 1) {
    log.resize(ls);
    n.nvrtcGetProgramLog_(prog, &log[0]);
  }
  if (log_out) *log_out = log;
  if (!env("B200_NVRTC_LOG").empty() && !log.empty()) fprintf(stderr, "[b200 nvrtc] %s: %s\n", name.c_str(), log.c_str());
  if (r != NVRTC_SUCCESS) {
    n.nvrtcDestroyProgram_(&prog);
    throw Error((int)r, "NVRTC failed to compile routine '" + name + "': " + n.nvrtcGetErrorString_(r) + "\n" + log);
  }
  size_t cs = 0;
  n.nvrtcGetCUBINSize_(prog, &cs);
  std::string cubin(cs, '\0');
  n.nvrtcGetCUBIN_(prog, &cubin[0]);
  n.nvrtcDestroyProgram_(&prog);
  std::lock_guard<std::mutex> g(mu);
  return cache.emplace(key, std::move(cubin)).first->second;
}

}  // namespace b200
