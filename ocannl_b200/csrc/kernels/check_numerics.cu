// Build-time check: the numeric prelude compiles for sm_100a and its helpers are usable
// from a kernel.
#include "numerics.cuh"

extern "C" __global__ void b200_check_numerics(const float* __restrict__ x, unsigned short* y, unsigned int* z, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  y[2 * i] = b200_f2bf(x[i]);
  y[2 * i + 1] = b200_f2h(b200_h2f(b200_f2h(x[i])) + b200_bf2f(y[2 * i]));
  b200_u4x32 k = b200_u32_widen((b200_u32)i), c = b200_u32_widen(42u);
  b200_u4x32 r = b200_threefry_light(k, c), s = b200_threefry_crypto(k, c);
  z[i] = r.v[0] ^ s.v[3];
  float w = b200_warp_sum(x[i]) + b200_warp_max(x[i]);
  if (w == 12345.f) z[i] = 0;
}
