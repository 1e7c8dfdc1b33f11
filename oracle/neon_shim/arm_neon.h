/*
 * Minimal <arm_neon.h> stand-in on GCC vector extensions (x86-64 host) -- TEST INFRASTRUCTURE.
 * Lets the reference's generated C artefacts (toolchain/generated/hermetic/ in the reference
 * tree), which are written against ARM NEON, compile and run on the test machine.  Covers exactly
 * the intrinsics those artefacts and the reference runtime header use; every lane operation is
 * the IEEE single-precision operation the NEON instruction performs (fused multiply-add through
 * fmaf, round-to-nearest-even through rintf).
 */
#ifndef DGEN_ORACLE_NEON_SHIM_H
#define DGEN_ORACLE_NEON_SHIM_H
#include <stdint.h>

typedef float float32x4_t __attribute__((vector_size(16)));
typedef uint32_t uint32x4_t __attribute__((vector_size(16)));
typedef int32_t int32x4_t __attribute__((vector_size(16)));
typedef float float32_t;

float fmaf(float, float, float);
float rintf(float);
float floorf(float);
float fabsf(float);

#define SHIM static inline __attribute__((always_inline, unused))

SHIM float32x4_t vdupq_n_f32(float v) { return (float32x4_t){v, v, v, v}; }
SHIM uint32x4_t vdupq_n_u32(uint32_t v) { return (uint32x4_t){v, v, v, v}; }
SHIM int32x4_t vdupq_n_s32(int32_t v) { return (int32x4_t){v, v, v, v}; }
SHIM float32x4_t vld1q_f32(const float *p) { float32x4_t r; __builtin_memcpy(&r, p, 16); return r; }
SHIM void vst1q_f32(float *p, float32x4_t v) { __builtin_memcpy(p, &v, 16); }
#define vgetq_lane_f32(v, lane) ((v)[lane])

SHIM float32x4_t vaddq_f32(float32x4_t a, float32x4_t b) { return a + b; }
SHIM float32x4_t vsubq_f32(float32x4_t a, float32x4_t b) { return a - b; }
SHIM float32x4_t vmulq_f32(float32x4_t a, float32x4_t b) { return a * b; }
SHIM float32x4_t vdivq_f32(float32x4_t a, float32x4_t b) { return a / b; }
SHIM float32x4_t vmulq_n_f32(float32x4_t a, float b) { return a * vdupq_n_f32(b); }
SHIM float32x4_t vnegq_f32(float32x4_t a) { return -a; }
SHIM float32x4_t vabsq_f32(float32x4_t a) {
  return (float32x4_t){fabsf(a[0]), fabsf(a[1]), fabsf(a[2]), fabsf(a[3])};
}
SHIM float32x4_t vminq_f32(float32x4_t a, float32x4_t b) {
  float32x4_t r; for (int i = 0; i < 4; ++i) r[i] = a[i] < b[i] ? a[i] : b[i]; return r;
}
SHIM float32x4_t vmaxq_f32(float32x4_t a, float32x4_t b) {
  float32x4_t r; for (int i = 0; i < 4; ++i) r[i] = a[i] > b[i] ? a[i] : b[i]; return r;
}
/* vfmaq_f32(a, b, c) = a + b*c ; vfmsq_f32(a, b, c) = a - b*c, single rounding */
SHIM float32x4_t vfmaq_f32(float32x4_t a, float32x4_t b, float32x4_t c) {
  float32x4_t r; for (int i = 0; i < 4; ++i) r[i] = fmaf(b[i], c[i], a[i]); return r;
}
SHIM float32x4_t vfmsq_f32(float32x4_t a, float32x4_t b, float32x4_t c) {
  float32x4_t r; for (int i = 0; i < 4; ++i) r[i] = fmaf(-b[i], c[i], a[i]); return r;
}
SHIM float32x4_t vrndmq_f32(float32x4_t a) {
  return (float32x4_t){floorf(a[0]), floorf(a[1]), floorf(a[2]), floorf(a[3])};
}
SHIM float32x4_t vrndnq_f32(float32x4_t a) {
  return (float32x4_t){rintf(a[0]), rintf(a[1]), rintf(a[2]), rintf(a[3])};
}

SHIM uint32x4_t vceqq_f32(float32x4_t a, float32x4_t b) { return (uint32x4_t)(a == b); }
SHIM uint32x4_t vcgtq_f32(float32x4_t a, float32x4_t b) { return (uint32x4_t)(a > b); }
SHIM uint32x4_t vcgeq_f32(float32x4_t a, float32x4_t b) { return (uint32x4_t)(a >= b); }
SHIM uint32x4_t vcltq_f32(float32x4_t a, float32x4_t b) { return (uint32x4_t)(a < b); }
SHIM uint32x4_t vcleq_f32(float32x4_t a, float32x4_t b) { return (uint32x4_t)(a <= b); }
SHIM uint32x4_t vceqq_u32(uint32x4_t a, uint32x4_t b) { return (uint32x4_t)(a == b); }
SHIM uint32x4_t vandq_u32(uint32x4_t a, uint32x4_t b) { return a & b; }
SHIM uint32x4_t vorrq_u32(uint32x4_t a, uint32x4_t b) { return a | b; }
SHIM uint32x4_t veorq_u32(uint32x4_t a, uint32x4_t b) { return a ^ b; }
SHIM uint32x4_t vmvnq_u32(uint32x4_t a) { return ~a; }
#define vshrq_n_u32(a, n) ((a) >> (n))
#define vshlq_n_u32(a, n) ((a) << (n))
SHIM int32x4_t vaddq_s32(int32x4_t a, int32x4_t b) { return a + b; }
SHIM int32x4_t vsubq_s32(int32x4_t a, int32x4_t b) { return a - b; }

SHIM uint32x4_t vreinterpretq_u32_f32(float32x4_t a) { return (uint32x4_t)a; }
SHIM float32x4_t vreinterpretq_f32_u32(uint32x4_t a) { return (float32x4_t)a; }
SHIM int32x4_t vreinterpretq_s32_u32(uint32x4_t a) { return (int32x4_t)a; }
SHIM uint32x4_t vreinterpretq_u32_s32(int32x4_t a) { return (uint32x4_t)a; }
/* NEON convert rounds toward zero */
SHIM int32x4_t vcvtq_s32_f32(float32x4_t a) {
  return (int32x4_t){(int32_t)a[0], (int32_t)a[1], (int32_t)a[2], (int32_t)a[3]};
}
SHIM float32x4_t vcvtq_f32_s32(int32x4_t a) {
  return (float32x4_t){(float)a[0], (float)a[1], (float)a[2], (float)a[3]};
}
SHIM float32x4_t vbslq_f32(uint32x4_t m, float32x4_t a, float32x4_t b) {
  return (float32x4_t)((m & (uint32x4_t)a) | (~m & (uint32x4_t)b));
}
SHIM float32x4_t vextq_f32(float32x4_t a, float32x4_t b, int n) {
  float t[8]; __builtin_memcpy(t, &a, 16); __builtin_memcpy(t + 4, &b, 16);
  return (float32x4_t){t[n], t[n + 1], t[n + 2], t[n + 3]};
}
#undef SHIM
#endif
