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
 *   - uniform conversions: builtins.c:345-360.
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

#endif
