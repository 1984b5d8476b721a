// b200_sum_f32_static: sum of a float range with NO allocation at call time.
//
// Who needs this: code that must not reach the device allocator while it runs — a caller
// inside a CUDA-graph capture or a latency-critical serving loop where cudaMalloc's implicit
// device synchronisation is unacceptable, a host thread that shares the GPU with a memory
// pool it must not fragment, or a process whose memory budget was handed out up front.  The
// routine path (b200_link) gets the scratch of its grid-wide reductions from cuMemAlloc; this
// entry point runs the same two-pass reduction (every block reduces a strided slice and
// writes one partial; one block combines the partials in block order) with the partials in a
// fixed array that lives in the library's device image instead.
//
// Limits and rules:
//   * the array holds B200_STATIC_MAX_BLOCKS (1024) partials = 4 KiB per GPU that loads the
//     library, held until the process exits;
//   * at most B200_STATIC_MAX_COUNT (2^26) elements per call; larger counts are refused with
//     B200_E_NO_SPACE before anything is launched; an empty range (count 0) writes 0.0f;
//   * both offsets must be multiples of 4 bytes (B200_E_INVALID otherwise, nothing is launched);
//   * a positive return value is the cudaError_t of the runtime call that failed;
//   * the first call on a device resolves the array's device address (cudaGetSymbolAddress,
//     with that device current).  Make that first call before starting any stream capture;
//   * every call on a device uses the same array.  Calls queued on the device's stream run one
//     after another and are safe; two calls that overlap on the GPU (other streams, other
//     host threads driving the same device) race on the partials.  Nothing in the array has
//     to start at zero: pass 1 overwrites exactly the slots pass 2 reads, so the previous
//     call's contents never leak into a result.
#include <cuda_runtime.h>

#include <mutex>

#include "runtime.hpp"

#define B200_STATIC_MAX_BLOCKS 1024
#define B200_STATIC_MAX_COUNT (1ull << 26)

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) float b200_static_partials[B200_STATIC_MAX_BLOCKS];

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* sh) {
  const unsigned int lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31u) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = lane < nwarps ? sh[lane] : 0.0f;
  return warp_sum(r);
}

__global__ void __launch_bounds__(1024) sum_pass1(const float* __restrict__ x, unsigned long long n, float* partials) {
  __shared__ float sh[32];
  float v = 0.0f;
  for (unsigned long long i = (unsigned long long)blockIdx.x * 1024ull + threadIdx.x; i < n;
       i += (unsigned long long)gridDim.x * 1024ull)
    v += x[i];
  v = block_sum(v, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = v;
}

__global__ void __launch_bounds__(256) sum_pass2(const float* partials, unsigned int blocks, float* out) {
  __shared__ float sh[32];
  float v = 0.0f;
  for (unsigned int i = threadIdx.x; i < blocks; i += blockDim.x) v += partials[i];
  v = block_sum(v, sh);
  if (threadIdx.x == 0) out[0] = v;
}

std::mutex g_setup_mu;
float* g_partials[64] = {nullptr};  // per device ordinal

}  // namespace

extern thread_local std::string b200_error_slot;  // api.cpp

extern "C" int b200_sum_f32_static(b200_dev* dev, int in_pool, size_t in_offset, size_t count, int out_pool,
                                   size_t out_offset) {
  try {
    if (!dev) throw b200::Error(B200_E_INVALID, "null device");
    if (dev->ordinal < 0 || dev->ordinal >= 64) throw b200::Error(B200_E_INVALID, "device ordinal out of range");
    // float accesses at an address that is not a multiple of 4 would fault on the device, and a
    // fault is sticky for the whole context: refuse on the host, before anything is launched
    if (in_offset % sizeof(float) != 0 || out_offset % sizeof(float) != 0)
      throw b200::Error(B200_E_INVALID, "b200_sum_f32_static: offsets must be multiples of 4 bytes");
    if ((unsigned long long)count > B200_STATIC_MAX_COUNT)
      throw b200::Error(B200_E_NO_SPACE, "b200_sum_f32_static: " + std::to_string(count) +
                                             " elements exceed the fixed capacity of " +
                                             std::to_string(B200_STATIC_MAX_COUNT) +
                                             " (the scratch array is static; use a routine for larger ranges)");
    dev->make_current();
    CUdeviceptr in = dev->address(in_pool, in_offset, count * sizeof(float));
    CUdeviceptr out = dev->address(out_pool, out_offset, sizeof(float));
    float* partials = nullptr;
    {
      std::lock_guard<std::mutex> g(g_setup_mu);
      if (!g_partials[dev->ordinal]) {
        // set-up, once per device, with that device current
        cudaError_t e = cudaSetDevice(dev->ordinal);
        if (e != cudaSuccess) throw b200::Error((int)e, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, b200_static_partials);
        if (e != cudaSuccess || !p)
          throw b200::Error((int)e, std::string("cudaGetSymbolAddress(b200_static_partials): ") + cudaGetErrorString(e));
        g_partials[dev->ordinal] = (float*)p;
      }
      partials = g_partials[dev->ordinal];
    }
    unsigned long long want = ((unsigned long long)count + 16383ull) / 16384ull;  // >= 16 elements per thread
    unsigned int blocks = (unsigned int)(want < 1 ? 1 : (want > B200_STATIC_MAX_BLOCKS ? B200_STATIC_MAX_BLOCKS : want));
    cudaStream_t s = (cudaStream_t)dev->stream;
    sum_pass1<<<blocks, 1024, 0, s>>>((const float*)in, (unsigned long long)count, partials);
    sum_pass2<<<1, 256, 0, s>>>(partials, blocks, (float*)out);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) throw b200::Error((int)e, std::string("b200_sum_f32_static launch: ") + cudaGetErrorString(e));
    dev->n_launches += 2;
    return 0;
  } catch (const b200::Error& e) {
    b200_error_slot = e.what();
    return e.code;
  } catch (const std::exception& e) {   // nothing may cross the C boundary
    b200_error_slot = e.what();
    return B200_E_INVALID;
  }
}
