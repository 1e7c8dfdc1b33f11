// Device helpers shared by the oscillator-bank forward and backward kernels: the reference's phasor
// recurrence, exact division by the sample rate, sampleRow positions, the centred fast sine.
#pragma once
#include "common.cuh"

namespace dgosc {

constexpr int CH = 64;            // frames per phase chunk
constexpr float TWO_PI_F = 6.2831850051879883f;  // Float(2*Float.pi) of the reference graphs

// a / b for a fixed b with r = RN(1/b): q + fma(-q, b, a) * r is the correctly rounded quotient
// (checked exhaustively on the host for the common sample rates, a in [1e-3, 2e6]).
__device__ __forceinline__ float div_by_const(float a, float b, float r) {
  float q = __fmul_rn(a, r);
  float rem = __fmaf_rn(-q, b, a);
  return __fmaf_rn(rem, r, q);
}

// One step of the reference recurrence: next = p + inc ; w = next - floor(next) ; if (w >= 1) w -= 1.
__device__ __forceinline__ float phasor_step(float p, float inc) {
  float next = __fadd_rn(p, inc);
  if (inc >= 0.0f && inc < 1.0f) {
    // p in [0,1) and inc in [0,1): next in [0,2), floor is 0 or 1 and next-1 is exact
    float t = __fadd_rn(next, -1.0f);
    return next >= 1.0f ? t : next;
  }
  float w = __fsub_rn(next, floorf(next));
  return w >= 1.0f ? __fadd_rn(w, -1.0f) : w;
}

// sampleRow position (Sources/DGen/Emit+RowSelection.swift:166-184)
__device__ __forceinline__ void row_pos(float idx, int rows, int &lo, int &hi, float &fr) {
  float fr_rows = (float)rows;
  float w = idx;
  if (!(idx >= 0.0f && idx < fr_rows)) {  // fmod is the identity inside [0, rows)
    w = fmodf(idx, fr_rows);
    if (w < 0.0f) w = __fadd_rn(w, fr_rows);
  }
  float fl = floorf(w);
  float ce = fl + 1.0f;
  if (ce >= fr_rows) ce = 0.0f;
  lo = (int)fl;
  hi = (int)ce;
  fr = __fsub_rn(w, fl);
}

__device__ __forceinline__ float lerp_strict(float omf, float a, float fr, float b) {
  return __fadd_rn(__fmul_rn(omf, a), __fmul_rn(fr, b));
}

// sin(2*pi*p) for p in [0,1): centre to [-pi, pi) where the fast sine's absolute error is 2^-21.4
__device__ __forceinline__ float sin_turns(float p) {
  float c = p >= 0.5f ? p - 1.0f : p;
  return __sinf(c * TWO_PI_F);
}
// -sin(2*pi*p) for p in [0,1) with a single subtraction for the centring: sin(2 pi p) = -sin(2 pi (p - 1/2)).
// p - 1/2 is exact for p >= 1/4 and within 2^-26 turns below, far inside the fast sine's own error.
__device__ __forceinline__ float neg_sin_turns(float p) { return __sinf(__fadd_rn(p, -0.5f) * TWO_PI_F); }
// (float)(j + 1 + step * i) for small integers without an integer-to-float conversion per use
__device__ __forceinline__ float partial_number(float kf0, int step_times_i) { return kf0 + (float)step_times_i; }

}  // namespace dgosc

// Runs the per-sample fundamental track and the phase-anchor kernels for `p` into `scratch`
// (dgc_harmonic_scratch_floats(p) floats); returns the control clock and the anchors [B][C][K].
// already_prepared: the scratch still holds the tracks and anchors of an earlier call with the same inputs;
// nothing is launched, only the pointers are returned.
// When uv_dev and gain_dev are given it also writes the per-sample output envelope
// env[b][n] = lerp(gain) * lerp(uv) * harmonic_scale, and in SCAN mode the anchors as Q0.32 turns.
// In FUNDAMENTAL mode no per-partial anchors exist (anchors_out is not written): extra->fund replaces them.
struct dgc_harmonic_extra {
  const float *f0t = nullptr;          // [B][T] per-sample fundamental
  const float *env = nullptr;          // [B][T] or nullptr
  const uint32_t *anchors_q = nullptr; // [B][C][K] (SCAN mode only) or nullptr
  const unsigned long long *fund = nullptr;  // [B][C] running sum of f0 / sr at every chunk start, Q0.64
                                             // (FUNDAMENTAL mode only): partial k starts chunk c at k * fund[b][c]
  const int2 *trk = nullptr;                 // [B][T] (FUNDAMENTAL mode only): x = the fundamental's phase advance from
                                             // the start of the frame's chunk in Q0.32, y = number of partials below
                                             // Nyquist at that frame
  float2 *sums = nullptr;                    // [B][T] (FUNDAMENTAL mode only): room for what the render divides per
                                             // frame, x = sum_k a_k sin(2 pi phi_k) / (sum_k a_k + eps), y = 1 / (sum_k
                                             // a_k + eps).  Written by a forward call that was given the scratch by
                                             // its caller (who keeps it for the backward); read by the backward that
                                             // is told the scratch is the forward's.
};
int32_t dgc_harmonic_prepare(dgc_ctx *ctx, const dgc_harmonic_params *p, const float *f0_dev, float *scratch,
                             const float **play_out, const float **anchors_out, const float *uv_dev = nullptr,
                             const float *gain_dev = nullptr, dgc_harmonic_extra *extra = nullptr,
                             bool already_prepared = false);
