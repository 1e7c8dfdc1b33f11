/*
 * CPU oracle for the frame-parallel render path -- TEST INFRASTRUCTURE, not product code.
 * Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may load it.
 *
 * Two instantiations of orc_impl.h: *_f32 (reference-C-backend-faithful single precision) and
 * *_f64 (double precision, gradient reference).  Pinned against (see tests/test_oracle_*.py):
 *   - the known-answer values of Tests/DGenLazyTests/CBackendTests.swift:46-76,
 *   - the four reference-generated C artefacts toolchain/generated/hermetic/*.c, compiled from
 *     where they lie by oracle/build_ref.sh into oracle/_ref/ (scalar phasor + polynomial
 *     sin/cos/tanh, history feedback + delay, bufferView ring + hop counter + Hann + FFT +
 *     partitioned MAC + IFFT + overlapAdd).
 * The spectral-loss forward has no reference test on the C backend: parity unpinned for that
 * function beyond this restatement of Sources/DGen/Emit+SpectralLoss.swift.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Swift's Float.pi is pi rounded toward zero (0x40490FDA = 3.14159250...), and 2*Float.pi is the
 * Float the generated code carries as 6.283185f (toolchain/generated/hermetic/scalar-synth.c:66). */
#define PI_CONST 3.1415925025939941
#define TWO_PI_CONST 6.2831850051879883

#define R float
#define SFX _f32
#define FLOOR floorf
#define FMOD fmodf
#define SIN sinf
#define COS cosf
#define SQRT sqrtf
#define LOG logf
#define FABS fabsf
#define POW powf
#include "orc_impl.h"
#undef R
#undef SFX
#undef FLOOR
#undef FMOD
#undef SIN
#undef COS
#undef SQRT
#undef LOG
#undef FABS
#undef POW

#undef TWO_PI_CONST
#undef PI_CONST
#define PI_CONST 3.14159265358979323846
#define TWO_PI_CONST 6.28318530717958647692
#define R double
#define SFX _f64
#define FLOOR floor
#define FMOD fmod
#define SIN sin
#define COS cos
#define SQRT sqrt
#define LOG log
#define FABS fabs
#define POW pow
#include "orc_impl.h"

/* Signal.noise(): xorshift32 (13,17,5); the state is a uint32 bit-stored in a float cell, a zero
 * state is reseeded to 1; value = state / 2^32.  Sources/DGen/Renderer/CRenderer.swift:660-695. */
void orc_noise_xorshift(uint32_t *state, int T, float *out) {
  uint32_t s = *state;
  for (int n = 0; n < T; ++n) {
    if (s == 0) s = 1;
    s ^= s << 13;
    s ^= s >> 17;
    s ^= s << 5;
    out[n] = (float)s / 4294967296.0f;
  }
  *state = s;
}

/* Output sanitiser: non-finite -> 0 (toolchain/include/dgen_runtime.h:72-74). */
void orc_sanitize(float *x, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    uint32_t bits;
    memcpy(&bits, &x[i], 4);
    if ((bits & 0x7f800000u) == 0x7f800000u) x[i] = 0.0f;
  }
}
