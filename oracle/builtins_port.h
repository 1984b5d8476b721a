/* CPU ORACLE helper header — test infrastructure only, never shipped or linked
 * into the device library.
 *
 * Restates, in plain C, the numeric helpers that the reference prepends to
 * every generated routine (arrayjit/lib/builtins_cc.ml, same arithmetic as
 * arrayjit/lib/builtins.c):
 *   - bfloat16 <-> float: builtins.c:611-627 (shift; round-to-nearest-even by
 *     adding 0x7FFF + lsb, no NaN special case);
 *   - half: native _Float16 when the compiler has it (builtins.c:11-21);
 *   - threefry4x32, 20-round and 2-round forms: builtins.c:156-329
 *     (Threefry-4x32 of Salmon et al., "Parallel random numbers: as easy as
 *     1, 2, 3", with the rotation pairs 13/15/26/6 and 17/29/16/24 applied as
 *     two mixes per call and a word swap after each);
 *   - uniform conversions, scalar and vector forms: builtins.c:345-528;
 *   - widening to uint4x32: builtins.c:531-606.
 * Checked bit for bit against the reference's builtins.c compiled into
 * oracle/_ref (tests/test_oracle_golden.py).
 */
#ifndef B200_ORACLE_BUILTINS_PORT_H
#define B200_ORACLE_BUILTINS_PORT_H

#include <stdio.h>
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <stdlib.h>

#ifdef __FLT16_MAX__
#define HALF_T _Float16
#define HALF_TO_FP(x) (x)
#define FP_TO_HALF(x) (x)
#define HALF_TO_FLOAT(x) ((float)(x))
#define FLOAT_TO_HALF(x) ((_Float16)(x))
#else
#error "the oracle expects a compiler with _Float16 (gcc >= 12 on x86-64)"
#endif

static inline float bfloat16_to_single(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t single_to_bfloat16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

typedef struct { uint32_t v[4]; } uint4x32_t;
typedef struct { float v[4]; } float4_t;
typedef struct { double v[2]; } double2_t;
typedef struct { int32_t v[4]; } int32x4_t;
typedef struct { int64_t v[2]; } int64x2_t;
typedef struct { uint16_t v[8]; } uint16x8_t;
typedef struct { HALF_T v[8]; } half8_t;

static inline uint32_t b200o_rotl(uint32_t x, unsigned n) { return (x << n) | (x >> (32 - n)); }

/* one call = two mix steps on (x0,x1),(x2,x3), swapping x1/x3 after each */
static inline void b200o_mix2(uint32_t x[4], unsigned r0, unsigned r1, unsigned r2, unsigned r3) {
  uint32_t t;
  x[0] += x[1]; x[1] = b200o_rotl(x[1], r0) ^ x[0];
  x[2] += x[3]; x[3] = b200o_rotl(x[3], r1) ^ x[2];
  t = x[1]; x[1] = x[3]; x[3] = t;
  x[0] += x[1]; x[1] = b200o_rotl(x[1], r2) ^ x[0];
  x[2] += x[3]; x[3] = b200o_rotl(x[3], r3) ^ x[2];
  t = x[1]; x[1] = x[3]; x[3] = t;
}

static inline uint4x32_t b200o_threefry(uint4x32_t key, uint4x32_t ctr, int injections) {
  uint32_t ks[5], x[4];
  int i, s;
  ks[4] = 0x1BD11BDAu;
  for (i = 0; i < 4; ++i) { ks[i] = key.v[i]; ks[4] ^= key.v[i]; x[i] = ctr.v[i] + key.v[i]; }
  for (s = 1; s <= injections; ++s) {
    b200o_mix2(x, 13, 15, 26, 6);
    b200o_mix2(x, 17, 29, 16, 24);
    if (injections > 1) {           /* the 20-round form does 4 calls between injections */
      b200o_mix2(x, 13, 15, 26, 6);
      b200o_mix2(x, 17, 29, 16, 24);
    }
    for (i = 0; i < 4; ++i) x[i] += ks[(s + i) % 5];
    x[3] += (uint32_t)s;
  }
  uint4x32_t r;
  for (i = 0; i < 4; ++i) r.v[i] = x[i];
  return r;
}

static inline uint4x32_t arrayjit_threefry4x32_crypto(uint4x32_t key, uint4x32_t ctr) {
  return b200o_threefry(key, ctr, 5);
}
static inline uint4x32_t arrayjit_threefry4x32_light(uint4x32_t key, uint4x32_t ctr) {
  return b200o_threefry(key, ctr, 1);
}

static inline float uint32_to_single_uniform(uint32_t x) {
  return (float)(x >> 8) * (1.0f / 16777216.0f);
}
static inline float uint4x32_to_single_uniform(uint4x32_t x) {
  return uint32_to_single_uniform(x.v[0]);
}
static inline float4_t uint4x32_to_single_uniform_vec(uint4x32_t x) {
  float4_t r;
  for (int i = 0; i < 4; ++i) r.v[i] = uint32_to_single_uniform(x.v[i]);
  return r;
}

/* integer -> uint4x32 widening: the value xor-ed with three odd constants / a half-word
 * rotation so that 2-round threefry sees four distinct words (builtins.c:545-578) */
static inline uint4x32_t uint32_to_uint4x32(uint32_t x) {
  uint4x32_t r = {{x, x ^ 0x9E3779B9u, x ^ 0x6C078965u, x ^ ((x << 16) | (x >> 16))}};
  return r;
}
static inline uint4x32_t int32_to_uint4x32(int32_t x) { return uint32_to_uint4x32((uint32_t)x); }
static inline uint4x32_t single_to_uint4x32(float f) {
  uint4x32_t r = {{0, 0, 0, 0}};
  memcpy(&r.v[0], &f, 4);
  return r;
}
/* 64-bit sources fill the two low words (builtins.c:538-543,559-563,579-582) */
static inline uint4x32_t uint64_to_uint4x32(uint64_t x) {
  uint4x32_t r = {{(uint32_t)(x & 0xFFFFFFFFu), (uint32_t)(x >> 32), 0, 0}};
  return r;
}
static inline uint4x32_t int64_to_uint4x32(int64_t x) { return uint64_to_uint4x32((uint64_t)x); }
static inline uint4x32_t double_to_uint4x32(double d) {
  uint64_t bits;
  memcpy(&bits, &d, 8);
  return uint64_to_uint4x32(bits);
}
/* 16-bit sources go to word 0 as they are (builtins.c:589-602) */
static inline uint4x32_t uint16_to_uint4x32(uint16_t x) {
  uint4x32_t r = {{(uint32_t)x, 0, 0, 0}};
  return r;
}
static inline uint4x32_t bfloat16_to_uint4x32(uint16_t x) { return uint16_to_uint4x32(x); }

/* ---- scalar uniform forms (builtins.c:351-414) */
static inline double uint4x32_to_double_uniform(uint4x32_t x) {
  uint64_t c = ((uint64_t)x.v[1] << 32) | x.v[0];
  return c * (1.0 / 18446744073709551616.0);
}
static inline int32_t uint4x32_to_int32_uniform(uint4x32_t x) { return (int32_t)x.v[0]; }
static inline uint32_t uint4x32_to_uint32_uniform(uint4x32_t x) { return x.v[0]; }
static inline int64_t uint4x32_to_int64_uniform(uint4x32_t x) {
  return (int64_t)(((uint64_t)x.v[1] << 32) | x.v[0]);
}
static inline uint16_t b200o_round_bits_bf16(float f) {
  /* round to nearest even written with guard / sticky tests (builtins.c:399-405) */
  uint32_t bits;
  memcpy(&bits, &f, 4);
  uint16_t bf = (uint16_t)(bits >> 16);
  if ((bits & 0x8000u) && ((bits & 0x7FFFu) || (bf & 1u))) bf++;
  return bf;
}
static inline uint16_t uint4x32_to_bfloat16_uniform(uint4x32_t x) {
  return b200o_round_bits_bf16(uint32_to_single_uniform(x.v[0]));
}
/* The reference declares this one `uint16_t` while returning FLOAT_TO_HALF(f); with a native
 * _Float16 that converts the VALUE (always 0).  The port returns the half itself, as the
 * vector form does (builtins.c:407-412 against :501-513). */
static inline HALF_T uint4x32_to_half_uniform(uint4x32_t x) {
  float f = (float)(x.v[0] & 0xFFFFu) * (1.0f / 65536.0f);
  return FLOAT_TO_HALF(f);
}

/* ---- vector uniform forms: all 128 bits are used (builtins.c:428-528) */
static inline double2_t uint4x32_to_double_uniform_vec(uint4x32_t x) {
  double2_t r;
  for (int i = 0; i < 2; ++i) {
    uint64_t c = ((uint64_t)x.v[2 * i + 1] << 32) | x.v[2 * i];
    r.v[i] = c * (1.0 / 18446744073709551616.0);
  }
  return r;
}
static inline int32x4_t uint4x32_to_int32_uniform_vec(uint4x32_t x) {
  int32x4_t r;
  for (int i = 0; i < 4; ++i) r.v[i] = (int32_t)x.v[i];
  return r;
}
static inline int64x2_t uint4x32_to_int64_uniform_vec(uint4x32_t x) {
  int64x2_t r;
  for (int i = 0; i < 2; ++i) r.v[i] = (int64_t)(((uint64_t)x.v[2 * i + 1] << 32) | x.v[2 * i]);
  return r;
}
static inline uint16x8_t uint4x32_to_bfloat16_uniform_vec(uint4x32_t x) {
  uint16x8_t r;
  for (int i = 0; i < 8; ++i) {
    uint32_t h = (x.v[i / 2] >> (16 * (i & 1))) & 0xFFFFu;
    r.v[i] = b200o_round_bits_bf16((float)h * (1.0f / 65536.0f));
  }
  return r;
}
static inline half8_t uint4x32_to_half_uniform_vec(uint4x32_t x) {
  half8_t r;
  for (int i = 0; i < 8; ++i) {
    uint32_t h = (x.v[i / 2] >> (16 * (i & 1))) & 0xFFFFu;
    r.v[i] = FLOAT_TO_HALF((float)h * (1.0f / 65536.0f));
  }
  return r;
}


/* ---- 8-bit floats, 1-5-2 (arrayjit/lib/builtins.c:643-742).  The reference's narrowing is restated
 * step for step, quirks included, because results must carry the same bits: the significand that
 * frexpf returns in [0.5, 1) is mapped to (m - 0.5) * 4 in [0, 2) and rounded by adding a half and
 * truncating, so only the codes with mantissa 0, 1 and 2 are ever produced for normal numbers, and
 * widening a code and narrowing it again is not always the identity (mantissa 2 comes back as 1). */
static inline float fp8_to_single(uint8_t c) {
  if (c == 0) return 0.0f;
  const uint32_t sign = (c >> 7) & 1u, e = (c >> 2) & 0x1Fu, m = c & 3u;
  float r;
  if (e == 0x1Fu) r = m == 0 ? INFINITY : NAN;
  else if (e == 0) r = ldexpf((float)m / 4.0f, -14);
  else r = (1.0f + (float)m * 0.25f) * ldexpf(1.0f, (int)e - 15);
  if (e == 0x1Fu && m != 0) return r;          /* NaN keeps no sign */
  return sign ? -r : r;
}
static inline uint8_t single_to_fp8(float f) {
  if (f == 0.0f) return 0;
  const uint32_t sign = f < 0 ? 1u : 0u;
  f = fabsf(f);
  if (isinf(f)) return (uint8_t)((sign << 7) | 0x7Cu);
  if (isnan(f)) return (uint8_t)((sign << 7) | 0x7Fu);
  int ex;
  float m = frexpf(f, &ex);
  const int e = ex + 14;
  if (e < 0) return (uint8_t)(sign << 7);
  if (e > 30) return (uint8_t)((sign << 7) | 0x7Cu);
  uint32_t bits;
  if (e == 0) {
    bits = (uint32_t)(f * ldexpf(1.0f, 14) * 4.0f + 0.5f);
    if (bits > 3u) bits = 3u;
    return (uint8_t)((sign << 7) | bits);
  }
  bits = (uint32_t)((m - 0.5f) * 4.0f + 0.5f);
  if (bits > 3u) bits = 3u;
  return (uint8_t)((sign << 7) | (((uint32_t)e & 0x1Fu) << 2) | bits);
}
typedef struct { uint8_t v[16]; } uint8x16_t;
static inline uint8_t uint4x32_to_fp8_uniform(uint4x32_t x) { return (uint8_t)(x.v[0] & 0xFFu); }
static inline uint8_t uint4x32_to_byte_uniform(uint4x32_t x) { return (uint8_t)(x.v[0] & 0xFFu); }
static inline uint8x16_t uint4x32_to_fp8_uniform_vec(uint4x32_t x) {
  uint8x16_t r;
  for (int i = 0; i < 16; ++i) r.v[i] = (uint8_t)(x.v[i / 4] >> (8 * (i % 4)));
  return r;
}
static inline uint4x32_t fp8_to_uint4x32(uint8_t x) { return uint16_to_uint4x32((uint16_t)x); }

#endif
