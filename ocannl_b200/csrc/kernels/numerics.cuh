// Device numerics shared by every generated kernel.  Self-contained (no headers) so that
// NVRTC can compile it as the prelude of a routine's translation unit.
//
// Bit-level helpers follow the reference's C helpers so that integer paths agree bit for
// bit with the cc backend (arrayjit/lib/builtins.c):
//   bf16 <-> f32        :611-627  (round to nearest even; same bits as the reference's
//                                  add-0x7FFF-plus-lsb formula for everything but NaN payloads)
//   threefry4x32        :156-329  (20-round and 2-round forms)
//   uniform conversions :345-360, widening to uint4x32 :545-578
// Half values are stored as their 16 bits; arithmetic on them is done in f32 and rounded
// once per operation, as arrayjit/lib/cc_backend.ml:169-322 prescribes.
#ifndef B200_NUMERICS_CUH
#define B200_NUMERICS_CUH

typedef unsigned int b200_u32;
typedef unsigned long long b200_u64;

#define B200_INF (__int_as_float(0x7f800000))
#define B200_NAN (__int_as_float(0x7fffffff))

__device__ __forceinline__ float b200_bf2f(unsigned short h) { return __uint_as_float(((b200_u32)h) << 16); }
// Round to nearest even in one instruction.  For every finite value and for infinities this is
// bit-identical to the reference's `(u + 0x7FFF + ((u >> 16) & 1)) >> 16`; NaNs come out as the
// canonical NaN instead of a truncated payload.
__device__ __forceinline__ unsigned short b200_f2bf(float f) {
#ifdef B200_F2BF_INT
  b200_u32 u = __float_as_uint(f);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (unsigned short)(u >> 16);
#endif
  unsigned short h;
  asm("{ .reg .b16 t; cvt.rn.bf16.f32 t, %1; mov.b16 %0, t; }" : "=h"(h) : "f"(f));
  return h;
}
__device__ __forceinline__ float b200_h2f(unsigned short h) {
  float f;
  asm("{ .reg .b16 t; mov.b16 t, %1; cvt.f32.f16 %0, t; }" : "=f"(f) : "h"(h));
  return f;
}
__device__ __forceinline__ unsigned short b200_f2h(float f) {
  unsigned short h;
  asm("{ .reg .b16 t; cvt.rn.f16.f32 t, %1; mov.b16 %0, t; }" : "=h"(h) : "f"(f));
  return h;
}

// 8-bit floats, 1-5-2 (arrayjit/lib/builtins.c:643-742).  The narrowing repeats the reference's steps
// one by one, because it is not a plain rounding: the significand frexpf returns in [0.5, 1) goes
// to (m - 0.5) * 4 in [0, 2), a half is added and the sum truncated, so normal numbers only ever
// get mantissa codes 0, 1, 2, and widening a code then narrowing it is not always the identity.
// An 8-bit value therefore travels through expressions as its CODE, never as a float.
__device__ __forceinline__ float b200_fp82f(unsigned char c) {
  if (c == 0) return 0.0f;
  const b200_u32 sign = (c >> 7) & 1u, e = (c >> 2) & 0x1Fu, m = c & 3u;
  if (e == 0x1Fu) return m == 0 ? (sign ? -B200_INF : B200_INF) : B200_NAN;
  const float r = e == 0 ? ldexpf((float)m / 4.0f, -14) : (1.0f + (float)m * 0.25f) * ldexpf(1.0f, (int)e - 15);
  return sign ? -r : r;
}
__device__ __forceinline__ unsigned char b200_f2fp8(float f) {
  if (f == 0.0f) return 0;
  const b200_u32 sign = f < 0 ? 1u : 0u;
  f = fabsf(f);
  if (isinf(f)) return (unsigned char)((sign << 7) | 0x7Cu);
  if (isnan(f)) return (unsigned char)((sign << 7) | 0x7Fu);
  int ex;
  const float m = frexpf(f, &ex);
  const int e = ex + 14;
  if (e < 0) return (unsigned char)(sign << 7);
  if (e > 30) return (unsigned char)((sign << 7) | 0x7Cu);
  b200_u32 bits;
  if (e == 0) {
    bits = (b200_u32)(f * 16384.0f * 4.0f + 0.5f);
    if (bits > 3u) bits = 3u;
    return (unsigned char)((sign << 7) | bits);
  }
  bits = (b200_u32)((m - 0.5f) * 4.0f + 0.5f);
  if (bits > 3u) bits = 3u;
  return (unsigned char)((sign << 7) | (((b200_u32)e & 0x1Fu) << 2) | bits);
}

// "Rounded floats": the value of a bf16 / half number kept in a float register.
__device__ __forceinline__ float b200_rbf(float f) {
  b200_u32 u;
  asm("cvt.rn.bf16x2.f32 %0, %1, %1;" : "=r"(u) : "f"(f));   // both halves hold bf16(f)
  return __uint_as_float(u & 0xFFFF0000u);
}
__device__ __forceinline__ float b200_rhf(float f) { return b200_h2f(b200_f2h(f)); }
// the 16 bits of a float that already holds a bf16 value
__device__ __forceinline__ unsigned short b200_bfbits(float f) { return (unsigned short)(__float_as_uint(f) >> 16); }
// two such floats as one 32-bit word (element 0 in the low half)
__device__ __forceinline__ b200_u32 b200_pack_bf(float lo, float hi) {
  return (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xFFFF0000u);
}
__device__ __forceinline__ b200_u32 b200_pack_hf(float lo, float hi) {
  return (b200_u32)b200_f2h(lo) | ((b200_u32)b200_f2h(hi) << 16);
}

// ---- pairs of neighbouring elements: two floats, or two 16-bit values in one word (the first
//      element in the low half).  The packed add / sub / mul round the exact result once, which
//      for operands of the 16-bit format equals the float operation followed by a rounding.
struct __align__(8) b200_f2 {
  float x, y;
};
__device__ __forceinline__ float b200_bf2_lo(b200_u32 v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float b200_bf2_hi(b200_u32 v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ float b200_hf2_lo(b200_u32 v) { return b200_h2f((unsigned short)(v & 0xFFFFu)); }
__device__ __forceinline__ float b200_hf2_hi(b200_u32 v) { return b200_h2f((unsigned short)(v >> 16)); }
__device__ __forceinline__ b200_u32 b200_bf2_pack(float lo, float hi) {
  b200_u32 u;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(u) : "f"(hi), "f"(lo));
  return u;
}
__device__ __forceinline__ b200_u32 b200_hf2_pack(float lo, float hi) {
  b200_u32 u;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(u) : "f"(hi), "f"(lo));
  return u;
}
__device__ __forceinline__ b200_u32 b200_dup16(unsigned short h) { return (b200_u32)h | ((b200_u32)h << 16); }
__device__ __forceinline__ b200_u32 b200_sel16x2(bool c0, bool c1, b200_u32 a, b200_u32 b) {
  return ((c0 ? a : b) & 0xFFFFu) | ((c1 ? a : b) & 0xFFFF0000u);
}
#define B200_PACKED_OP(NAME, PTX)                                                   \
  __device__ __forceinline__ b200_u32 NAME(b200_u32 a, b200_u32 b) {               \
    b200_u32 d;                                                                     \
    asm(PTX " %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));                             \
    return d;                                                                       \
  }
B200_PACKED_OP(b200_bf2_add, "add.rn.bf16x2")
B200_PACKED_OP(b200_bf2_sub, "sub.rn.bf16x2")
B200_PACKED_OP(b200_bf2_mul, "mul.rn.bf16x2")
B200_PACKED_OP(b200_bf2_max, "max.bf16x2")
B200_PACKED_OP(b200_bf2_min, "min.bf16x2")
B200_PACKED_OP(b200_hf2_add, "add.rn.f16x2")
B200_PACKED_OP(b200_hf2_sub, "sub.rn.f16x2")
B200_PACKED_OP(b200_hf2_mul, "mul.rn.f16x2")
B200_PACKED_OP(b200_hf2_max, "max.f16x2")
B200_PACKED_OP(b200_hf2_min, "min.f16x2")

__device__ __forceinline__ float b200_pow2(float x) { return x * x; }
__device__ __forceinline__ float b200_pow3(float x) { return x * x * x; }
__device__ __forceinline__ double b200_pow2(double x) { return x * x; }
__device__ __forceinline__ double b200_pow3(double x) { return x * x * x; }
__device__ __forceinline__ float b200_tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ b200_u32 b200_bits32(float f) { return __float_as_uint(f); }
__device__ __forceinline__ b200_u32 b200_bits32(b200_u32 u) { return u; }
__device__ __forceinline__ b200_u32 b200_bits32(int i) { return (b200_u32)i; }

struct b200_u4x32 {
  b200_u32 v[4];
};

__device__ __forceinline__ b200_u32 b200_rotl(b200_u32 x, unsigned n) { return (x << n) | (x >> (32 - n)); }
__device__ __forceinline__ void b200_mix2(b200_u32* x, unsigned r0, unsigned r1, unsigned r2, unsigned r3) {
  b200_u32 t;
  x[0] += x[1]; x[1] = b200_rotl(x[1], r0) ^ x[0];
  x[2] += x[3]; x[3] = b200_rotl(x[3], r1) ^ x[2];
  t = x[1]; x[1] = x[3]; x[3] = t;
  x[0] += x[1]; x[1] = b200_rotl(x[1], r2) ^ x[0];
  x[2] += x[3]; x[3] = b200_rotl(x[3], r3) ^ x[2];
  t = x[1]; x[1] = x[3]; x[3] = t;
}
template <int INJECTIONS>
__device__ __forceinline__ b200_u4x32 b200_threefry(b200_u4x32 key, b200_u4x32 ctr) {
  b200_u32 ks[5], x[4];
  ks[4] = 0x1BD11BDAu;
#pragma unroll
  for (int i = 0; i < 4; ++i) { ks[i] = key.v[i]; ks[4] ^= key.v[i]; x[i] = ctr.v[i] + key.v[i]; }
#pragma unroll
  for (int s = 1; s <= INJECTIONS; ++s) {
    b200_mix2(x, 13, 15, 26, 6);
    b200_mix2(x, 17, 29, 16, 24);
    if (INJECTIONS > 1) {
      b200_mix2(x, 13, 15, 26, 6);
      b200_mix2(x, 17, 29, 16, 24);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] += ks[(s + i) % 5];
    x[3] += (b200_u32)s;
  }
  b200_u4x32 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = x[i];
  return r;
}
__device__ __forceinline__ b200_u4x32 b200_threefry_crypto(b200_u4x32 k, b200_u4x32 c) { return b200_threefry<5>(k, c); }
__device__ __forceinline__ b200_u4x32 b200_threefry_light(b200_u4x32 k, b200_u4x32 c) { return b200_threefry<1>(k, c); }
__device__ __forceinline__ float b200_u32_uniform(b200_u32 x) { return (float)(x >> 8) * (1.0f / 16777216.0f); }
__device__ __forceinline__ b200_u4x32 b200_u32_widen(b200_u32 x) {
  b200_u4x32 r;
  r.v[0] = x; r.v[1] = x ^ 0x9E3779B9u; r.v[2] = x ^ 0x6C078965u; r.v[3] = x ^ ((x << 16) | (x >> 16));
  return r;
}

// widening of the other sources (arrayjit/lib/builtins.c:531-606)
__device__ __forceinline__ b200_u4x32 b200_u64_to_u4x32(b200_u64 x) {
  b200_u4x32 r;
  r.v[0] = (b200_u32)(x & 0xFFFFFFFFull); r.v[1] = (b200_u32)(x >> 32); r.v[2] = 0u; r.v[3] = 0u;
  return r;
}
__device__ __forceinline__ b200_u4x32 b200_f64_to_u4x32(double d) { return b200_u64_to_u4x32((b200_u64)__double_as_longlong(d)); }
__device__ __forceinline__ b200_u4x32 b200_word_to_u4x32(b200_u32 x) {
  b200_u4x32 r;
  r.v[0] = x; r.v[1] = 0u; r.v[2] = 0u; r.v[3] = 0u;
  return r;
}
__device__ __forceinline__ b200_u4x32 b200_f32_to_u4x32(float f) { return b200_word_to_u4x32(__float_as_uint(f)); }

// uniform values from random bits: element i of the vector forms (builtins.c:428-528) and the
// scalar forms (builtins.c:351-414).  16-bit results are returned as storage bits.
__device__ __forceinline__ unsigned short b200_bf16_bits_rne(float f) {
  const b200_u32 bits = __float_as_uint(f);
  unsigned short bf = (unsigned short)(bits >> 16);
  if ((bits & 0x8000u) && ((bits & 0x7FFFu) || (bf & 1u))) bf++;
  return bf;
}
__device__ __forceinline__ float b200_uniform_single(b200_u4x32 x, int i) { return b200_u32_uniform(x.v[i]); }
__device__ __forceinline__ double b200_uniform_double(b200_u4x32 x, int i) {
  const b200_u64 c = ((b200_u64)x.v[2 * i + 1] << 32) | x.v[2 * i];
  return (double)c * (1.0 / 18446744073709551616.0);
}
__device__ __forceinline__ int b200_uniform_int32(b200_u4x32 x, int i) { return (int)x.v[i]; }
__device__ __forceinline__ long long b200_uniform_int64(b200_u4x32 x, int i) {
  return (long long)(((b200_u64)x.v[2 * i + 1] << 32) | x.v[2 * i]);
}
__device__ __forceinline__ float b200_uniform_16(b200_u4x32 x, int i) {
  return (float)((x.v[i >> 1] >> (16 * (i & 1))) & 0xFFFFu) * (1.0f / 65536.0f);
}
__device__ __forceinline__ unsigned short b200_uniform_bfloat16(b200_u4x32 x, int i) { return b200_bf16_bits_rne(b200_uniform_16(x, i)); }
__device__ __forceinline__ unsigned short b200_uniform_half(b200_u4x32 x, int i) { return b200_f2h(b200_uniform_16(x, i)); }
__device__ __forceinline__ unsigned short b200_uniform1_bfloat16(b200_u4x32 x) { return b200_bf16_bits_rne(b200_u32_uniform(x.v[0])); }

// byte i of the 16 bytes of a uint4x32 (arrayjit/lib/builtins.c:518-528: the 8-bit "uniform" values)
__device__ __forceinline__ unsigned char b200_uniform_byte(b200_u4x32 x, int i) {
  return (unsigned char)(x.v[i >> 2] >> (8 * (i & 3)));
}

// ---- a lane's share of a row: N consecutive elements, moved with the widest accesses their size
//      allows (16, 8 or 4 bytes; the caller guarantees that alignment).  Values of the 16-bit
//      formats are widened to the floats that hold them inside expressions.
template <int BYTES>
__device__ __forceinline__ void b200_ld_words(const void* p, b200_u32* w) {
  if constexpr (BYTES % 16 == 0) {
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) {
      const uint4 q = ((const uint4*)p)[i];
      w[4 * i] = q.x; w[4 * i + 1] = q.y; w[4 * i + 2] = q.z; w[4 * i + 3] = q.w;
    }
  } else if constexpr (BYTES % 8 == 0) {
#pragma unroll
    for (int i = 0; i < BYTES / 8; ++i) {
      const uint2 q = ((const uint2*)p)[i];
      w[2 * i] = q.x; w[2 * i + 1] = q.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < BYTES / 4; ++i) w[i] = ((const b200_u32*)p)[i];
  }
}
template <int BYTES>
__device__ __forceinline__ void b200_st_words(void* p, const b200_u32* w) {
  if constexpr (BYTES % 16 == 0) {
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) ((uint4*)p)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
  } else if constexpr (BYTES % 8 == 0) {
#pragma unroll
    for (int i = 0; i < BYTES / 8; ++i) ((uint2*)p)[i] = make_uint2(w[2 * i], w[2 * i + 1]);
  } else {
#pragma unroll
    for (int i = 0; i < BYTES / 4; ++i) ((b200_u32*)p)[i] = w[i];
  }
}
template <int N>
__device__ __forceinline__ void b200_ld_row(const float* p, float* r) {
  b200_u32 w[N];
  b200_ld_words<4 * N>(p, w);
#pragma unroll
  for (int i = 0; i < N; ++i) r[i] = __uint_as_float(w[i]);
}
template <int N>
__device__ __forceinline__ void b200_st_row(float* p, const float* r) {
  b200_u32 w[N];
#pragma unroll
  for (int i = 0; i < N; ++i) w[i] = __float_as_uint(r[i]);
  b200_st_words<4 * N>(p, w);
}
// 16-bit rows: `half` chooses the format
template <int N, bool HALF>
__device__ __forceinline__ void b200_ld_row16(const unsigned short* p, float* r) {
  b200_u32 w[N / 2];
  b200_ld_words<2 * N>(p, w);
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {
    if constexpr (HALF) {
      r[2 * i] = b200_h2f((unsigned short)w[i]);
      r[2 * i + 1] = b200_h2f((unsigned short)(w[i] >> 16));
    } else {
      r[2 * i] = __uint_as_float(w[i] << 16);
      r[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
}
template <int N, bool HALF>
__device__ __forceinline__ void b200_st_row16(unsigned short* p, const float* r) {
  b200_u32 w[N / 2];
#pragma unroll
  for (int i = 0; i < N / 2; ++i) w[i] = HALF ? b200_pack_hf(r[2 * i], r[2 * i + 1]) : b200_pack_bf(r[2 * i], r[2 * i + 1]);
  b200_st_words<2 * N>(p, w);
}

// Rows whose elements are dealt to the lanes four at a time: lane l owns elements
// (k * 32 + l) * 4 + j  (j < 4, k < N / 4), register e = 4 k + j.  Every access of a warp then
// covers one contiguous stretch of the row (512 bytes of floats, 256 bytes of 16-bit values)
// instead of 32 pieces a lane's share apart.
template <int N>
__device__ __forceinline__ void b200_ld_rowv(const float* p, unsigned int lane, float* r) {
#pragma unroll
  for (int k = 0; k < N / 4; ++k) {
    const uint4 q = ((const uint4*)p)[k * 32 + lane];
    r[4 * k] = __uint_as_float(q.x); r[4 * k + 1] = __uint_as_float(q.y);
    r[4 * k + 2] = __uint_as_float(q.z); r[4 * k + 3] = __uint_as_float(q.w);
  }
}
template <int N>
__device__ __forceinline__ void b200_st_rowv(float* p, unsigned int lane, const float* r) {
#pragma unroll
  for (int k = 0; k < N / 4; ++k)
    ((uint4*)p)[k * 32 + lane] = make_uint4(__float_as_uint(r[4 * k]), __float_as_uint(r[4 * k + 1]), __float_as_uint(r[4 * k + 2]),
                                            __float_as_uint(r[4 * k + 3]));
}
template <int N, bool HALF>
__device__ __forceinline__ void b200_ld_rowv16(const unsigned short* p, unsigned int lane, float* r) {
#pragma unroll
  for (int k = 0; k < N / 4; ++k) {
    const uint2 q = ((const uint2*)p)[k * 32 + lane];
    if constexpr (HALF) {
      r[4 * k] = b200_h2f((unsigned short)q.x); r[4 * k + 1] = b200_h2f((unsigned short)(q.x >> 16));
      r[4 * k + 2] = b200_h2f((unsigned short)q.y); r[4 * k + 3] = b200_h2f((unsigned short)(q.y >> 16));
    } else {
      r[4 * k] = __uint_as_float(q.x << 16); r[4 * k + 1] = __uint_as_float(q.x & 0xFFFF0000u);
      r[4 * k + 2] = __uint_as_float(q.y << 16); r[4 * k + 3] = __uint_as_float(q.y & 0xFFFF0000u);
    }
  }
}
template <int N, bool HALF>
__device__ __forceinline__ void b200_st_rowv16(unsigned short* p, unsigned int lane, const float* r) {
#pragma unroll
  for (int k = 0; k < N / 4; ++k) {
    uint2 q;
    q.x = HALF ? b200_pack_hf(r[4 * k], r[4 * k + 1]) : b200_pack_bf(r[4 * k], r[4 * k + 1]);
    q.y = HALF ? b200_pack_hf(r[4 * k + 2], r[4 * k + 3]) : b200_pack_bf(r[4 * k + 2], r[4 * k + 3]);
    ((uint2*)p)[k * 32 + lane] = q;
  }
}

// IEEE single-precision division.  A zero over a finite non-zero value is a signed zero; giving
// the division sequence a numerator of one in that case (and selecting the zero afterwards) keeps
// such lanes -- the masked entries of a softmax row -- off the sequence's slow path, which the whole
// warp would otherwise wait for.  No branch: neighbouring divisions still overlap.
__device__ __forceinline__ float b200_fdiv(float a, float b) {
  const bool zero = a == 0.0f && b != 0.0f && b == b;
  const float q = (zero ? 1.0f : a) / b;
  return zero ? a * copysignf(1.0f, b) : q;
}
// One divisor for many numerators (a softmax row's sum).  With r = RN(1 / b): q0 = RN(a r) is within
// one unit in the last place of a / b, the remainder a - q0 b is exact in one fused multiply-add, and
// RN(q0 + remainder r) is the correctly rounded quotient (Markstein's correction step, the one the
// division sequence itself uses) as long as nothing overflows or falls below the normal range;
// quotients below the normal range may differ in their last place.  Divisors outside [2^-60, 2^60]
// take the plain division.
struct b200_divisor {
  float b, r;
  bool fast;
};
__device__ __forceinline__ b200_divisor b200_divisor_of(float b) {
  b200_divisor d;
  d.b = b;
  d.r = 1.0f / b;
  const float m = fabsf(b);
  d.fast = m >= 0x1p-60f && m <= 0x1p+60f;
  return d;
}
// the short sequence; the caller has checked d.fast
__device__ __forceinline__ float b200_div_by(float a, const b200_divisor& d) {
  const float q0 = a * d.r;
  const float rem = fmaf(-q0, d.b, a);
  const float q = fmaf(rem, d.r, q0);
  return fabsf(q0) == B200_INF ? q0 : q;   // an infinite numerator (or an overflow) stays infinite
}

// ---- range-checked node accesses (routines compiled with bounds=1).  The proxy stands where the
//      node's pointer stood: node[i] with i outside the node records (code 2, node id, index) in the
//      device status word and lands on a sink instead of memory the node does not own.
__device__ unsigned long long b200_sink_words[4];
template <typename T>
struct b200_checked {
  T* p;
  unsigned long long n;
  unsigned int* status;
  unsigned int node;
  __device__ __forceinline__ T& operator[](unsigned long long i) const {
    if (i < n) return p[i];
    if (atomicCAS(status, 0u, 2u) == 0u) {
      status[1] = node;
      status[2] = (unsigned int)i;
      status[3] = (unsigned int)(i >> 32);
      __threadfence_system();
    }
    return *(T*)b200_sink_words;
  }
  __device__ __forceinline__ T* operator+(unsigned long long i) const { return &(*this)[i]; }
};

// ---- warp-level combine used by cooperative (one warp per output element) reductions
__device__ __forceinline__ float b200_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float b200_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float b200_warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ double b200_warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- block-level combine (one block per output element).  `sh` holds one slot per warp;
//      every thread of the block calls these together and every thread gets the result.
#define B200_BLOCK_REDUCE(NAME, T, WARP_FN, NEUTRAL)                              \
  __device__ __forceinline__ T NAME(T v, double* sh_raw) {                        \
    T* sh = (T*)sh_raw;                                                           \
    const unsigned int lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;         \
    const unsigned int nwarps = (blockDim.x + 31u) >> 5;                          \
    v = WARP_FN(v);                                                               \
    __syncthreads();                                                              \
    if (lane == 0) sh[warp] = v;                                                  \
    __syncthreads();                                                              \
    T r = lane < nwarps ? sh[lane] : (T)(NEUTRAL);                                \
    r = WARP_FN(r);                                                               \
    return r;                                                                     \
  }
B200_BLOCK_REDUCE(b200_block_sum, float, b200_warp_sum, 0.0f)
B200_BLOCK_REDUCE(b200_block_max, float, b200_warp_max, -B200_INF)
B200_BLOCK_REDUCE(b200_block_min, float, b200_warp_min, B200_INF)
B200_BLOCK_REDUCE(b200_block_sum, double, b200_warp_sum, 0.0)

#endif  // B200_NUMERICS_CUH
