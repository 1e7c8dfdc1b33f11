// Oscillator bank: scalar clocks, phase anchors (serial or prefix-scan) and the fused
// phase -> sin -> amplitude -> sum-over-partials render.
//
// Time axis decomposition.  The reference's stateful phasor adds f/sr and wraps once per sample in
// single precision (Sources/DGen/Emit+State.swift:322-369); every add rounds, and those roundings
// are part of the result.  The render kernel therefore follows that recurrence literally, but only
// inside chunks of CH = 64 frames: one thread-group per (voice, chunk) starts from a phase anchor
// and steps 64 times.  Anchors come from one of two kernels:
//   SEQUENTIAL  one thread per (voice, partial) runs the recurrence over all T frames and records
//               the state every 64 frames: bit-identical to the reference, latency bound;
//   SCAN        every (voice, partial, chunk) sums its 64 increments exactly in 64-bit fixed point,
//               a second kernel prefix-sums the chunk totals: frame-parallel.
#include "osc_common.cuh"

namespace {

using namespace dgosc;

// ---------------------------------------------------------------------------------------------
// scalar accum clock, one thread (Sources/DGen/Definitions.swift:215-246)
// ---------------------------------------------------------------------------------------------
__global__ void clock_accum_kernel(float incr, float mn, float mx, float state0, int T, float *out, int clip,
                                   float clip_lo, float clip_hi) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  float acc = state0;
  const float span = __fsub_rn(mx, mn);
  for (int n = 0; n < T; ++n) {
    float v = acc;
    if (clip) v = fminf(fmaxf(v, clip_lo), clip_hi);
    out[n] = v;
    float next = __fadd_rn(acc, incr);
    float rel = __fsub_rn(next, mn);
    float k = floorf(__fdiv_rn(rel, span));
    float w = __fsub_rn(next, __fmul_rn(k, span));
    acc = w >= mx ? __fsub_rn(w, span) : w;
  }
}

// ---------------------------------------------------------------------------------------------
// constant-frequency bank summed to mono
// ---------------------------------------------------------------------------------------------
// deterministic phasor: frame-parallel, one thread per frame looping over partials
__global__ void osc_const_det_kernel(const float *__restrict__ freq, const float *__restrict__ amp, int K, int T,
                                     float sr, float *__restrict__ audio) {
  extern __shared__ float sh[];  // inc[K], amp[K]
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    sh[k] = __fdiv_rn(freq[k], sr);
    sh[K + k] = amp[k];
  }
  __syncthreads();
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= T) return;
  float fn = (float)n, acc = 0.0f;
  for (int k = 0; k < K; ++k) {
    float raw = __fmul_rn(sh[k], fn);
    float p = __fsub_rn(raw, floorf(raw));
    acc += sin_turns(p) * sh[K + k];
  }
  audio[n] = acc;
}

// stateful phasor, constant frequency: anchors by the serial recurrence (one thread per partial)
__global__ void osc_const_anchor_seq_kernel(const float *__restrict__ freq, int K, int T, float sr,
                                            float *__restrict__ anchors /* [C][K] */) {
  int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= K) return;
  float inc = __fdiv_rn(freq[k], sr);
  float p = 0.0f;
  for (int n = 0; n < T; ++n) {
    if ((n & (CH - 1)) == 0) anchors[(size_t)(n / CH) * K + k] = p;
    p = phasor_step(p, inc);
  }
}

__global__ void osc_const_render_kernel(const float *__restrict__ freq, const float *__restrict__ amp,
                                        const float *__restrict__ anchors, int K, int T, float sr,
                                        float *__restrict__ audio) {
  // one warp per chunk; lanes stride over partials and keep 64 per-frame sums in registers; the
  // cross-lane sum is a fixed shuffle tree, so the result does not depend on scheduling
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  int C = (T + CH - 1) / CH;
  if (warp >= C) return;
  int n0 = warp * CH;
  float acc[CH];
#pragma unroll
  for (int s = 0; s < CH; ++s) acc[s] = 0.0f;
  for (int k = lane; k < K; k += 32) {
    float inc = __fdiv_rn(freq[k], sr), a = amp[k];
    float p = anchors[(size_t)warp * K + k];
#pragma unroll
    for (int s = 0; s < CH; ++s) {
      acc[s] = fmaf(sin_turns(p), a, acc[s]);
      p = phasor_step(p, inc);
    }
  }
#pragma unroll
  for (int s = 0; s < CH; ++s) {
    float v = acc[s];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == (s & 31) && n0 + s < T) audio[n0 + s] = v;
  }
}

// ---------------------------------------------------------------------------------------------
// batched harmonic bank
// ---------------------------------------------------------------------------------------------
// per-frame sampleRow position of the cached control clock: (floor row as int bits, fraction).
// Entry T (one past the frames) holds, as int bits in .x, the first frame whose floor row is below its
// predecessor's (the control clock wrapped), or a value above every frame index when the rows only ascend:
// preset by the host, lowered here with an atomic minimum.
__global__ void row_table_kernel(const float *__restrict__ play, int T, int F, float2 *__restrict__ tab) {
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= T) return;
  int lo, hi;
  float fr;
  row_pos(play[n], F, lo, hi, fr);
  tab[n] = make_float2(__int_as_float(lo), fr);
  if (n > 0) {
    int plo, phi;
    float pfr;
    row_pos(play[n - 1], F, plo, phi, pfr);
    if (lo < plo) atomicMin(reinterpret_cast<int *>(&tab[T].x), n);
  }
}

// f0t[b][n] = sampleRow(f0)[n][b], strict single-precision lerp; optionally the output envelope
// env[b][n] = lerp(gain) * lerp(uv) * scale
__global__ void f0_track_kernel(const float2 *__restrict__ rowtab, const float *__restrict__ f0, int B, int T, int F,
                                float *__restrict__ f0t, const float *__restrict__ uv,
                                const float *__restrict__ gain, float scale, float *__restrict__ env) {
  int n = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (n >= T) return;
  const float2 rt = rowtab[n];
  const int lo = __float_as_int(rt.x), hi = lo + 1 >= F ? 0 : lo + 1;
  const float fr = rt.y;
  float omf = __fsub_rn(1.0f, fr);
  f0t[(size_t)b * T + n] = lerp_strict(omf, f0[(size_t)lo * B + b], fr, f0[(size_t)hi * B + b]);
  if (env) {
    const float gt = fmaf(fr, gain[(size_t)hi * B + b], omf * gain[(size_t)lo * B + b]);
    const float uvt = fmaf(fr, uv[(size_t)hi * B + b], omf * uv[(size_t)lo * B + b]);
    env[(size_t)b * T + n] = gt * uvt * scale;
  }
}

// SEQUENTIAL anchors: thread = (voice, partial), partial fastest; anchors[b][c][k]
__global__ void anchor_seq_kernel(const float *__restrict__ f0t, int B, int T, int K, float sr, float rsr,
                                  float *__restrict__ anchors) {
  int lane_id = blockIdx.x * blockDim.x + threadIdx.x;
  if (lane_id >= B * K) return;
  int b = lane_id / K, k = lane_id - b * K;
  const float kf = (float)(k + 1);
  const float *f = f0t + (size_t)b * T;
  const int C = (T + CH - 1) / CH;
  float *out = anchors + (size_t)b * C * K + k;
  float p = 0.0f;
  for (int c = 0; c < C; ++c) {
    out[(size_t)c * K] = p;
    int n0 = c * CH, n1 = min(T, n0 + CH);
#pragma unroll 8
    for (int n = n0; n < n1; ++n) {
      float inc = div_by_const(__fmul_rn(kf, f[n]), sr, rsr);
      p = phasor_step(p, inc);
    }
  }
}

// Exact conversion of a float in [0,1) to Q0.64 with integer operations (bits below 2^-64 dropped).
__device__ __forceinline__ unsigned long long turns_to_q64(float v) {
  unsigned u = __float_as_uint(v);
  int e = (int)(u >> 23);                       // biased exponent (sign is 0)
  if (e == 0) return 0ull;                      // zero / subnormal: below 2^-64 anyway
  unsigned long long m = (unsigned long long)((u & 0x7fffffu) | 0x800000u);
  int sh = e - 86;                              // value = m * 2^(e-150); Q0.64 = m * 2^(e-86)
  return sh >= 0 ? (m << sh) : (sh > -24 ? (m >> (-sh)) : 0ull);
}

// SCAN anchors, stage 1: exact sum of the 64 increments of a chunk in Q0.64 (mod 1).
// Same thread mapping as the render kernel: a group of LPC lanes owns one (voice, chunk), lane j
// carries partials j, j+LPC, ... so the per-frame work (f0 load, loop) is shared by P partials.
template <int LPC, int P>
__global__ void __launch_bounds__(128)
anchor_sum_kernel(const float *__restrict__ f0t, int B, int T, int K, float sr, float rsr,
                  unsigned long long *__restrict__ sums /* [B][C][K] */) {
  constexpr int G = 128 / LPC;
  const int C = (T + CH - 1) / CH;
  const int g = threadIdx.x / LPC, j = threadIdx.x % LPC;
  const int c = blockIdx.x * G + g, b = blockIdx.y;
  if (c >= C) return;
  const float *f = f0t + (size_t)b * T;
  const int n0 = c * CH, n1 = min(T, n0 + CH);
  // Double-float accumulation: the 64 increments of a chunk are summed to ~2^-36 absolute, far below the
  // 2^-25 spacing of the single-precision anchors, with plain FP32 adds; the chunk total is converted to
  // Q0.64 once.  hi starts at 8.0 (an integer number of turns, invisible mod 1) so that |hi| >= |inc|
  // holds for every add of an increment below 8 turns and the three-operation Fast2Sum is error-free.
  // Increments of 1 turn and more (partials above the sample rate, far above Nyquist and masked, but their
  // phase must stay defined for when f0 comes down again) are summed unwrapped: only the sum mod 1 matters.
  float hi[P], lo[P];
#pragma unroll
  for (int i = 0; i < P; ++i) {
    hi[i] = 8.0f;
    lo[i] = 0.0f;
  }
  const float kmax = (float)K, kf0 = (float)(j + 1);
  for (int n = n0; n < n1; ++n) {
    const float f0 = f[n];
    // one decision per frame, taken as a branch: all increments of this frame in [0, 8)?
    if (f0 >= 0.0f && __fmul_rn(kmax, f0) < 8.0f * sr) {
#pragma unroll
      for (int i = 0; i < P; ++i) {
        const float inc = div_by_const(__fmul_rn(partial_number(kf0, LPC * i), f0), sr, rsr);
        const float s = __fadd_rn(hi[i], inc);
        lo[i] = __fadd_rn(lo[i], __fsub_rn(inc, __fsub_rn(s, hi[i])));
        hi[i] = s;
      }
    } else {
#pragma unroll
      for (int i = 0; i < P; ++i) {
        float inc = div_by_const(__fmul_rn(partial_number(kf0, LPC * i), f0), sr, rsr);
        if (!(inc >= 0.0f && inc < 1.0f)) inc = inc - floorf(inc);
        if (!(inc >= 0.0f && inc < 1.0f)) inc = 0.0f;  // non-finite or rounded up to 1
        const float s = __fadd_rn(hi[i], inc);
        lo[i] = __fadd_rn(lo[i], __fsub_rn(inc, __fsub_rn(s, hi[i])));
        hi[i] = s;
      }
    }
  }
  unsigned long long acc[P];
#pragma unroll
  for (int i = 0; i < P; ++i) {
    // hi in [8, 520], |lo| < 1e-2: total mod 1 in Q0.64 (two's-complement add handles a negative lo)
    float ip = floorf(hi[i]);
    unsigned long long q = turns_to_q64(__fsub_rn(hi[i], ip));
    float al = fabsf(lo[i]);
    unsigned long long ql = al < 1.0f ? turns_to_q64(al) : 0ull;
    acc[i] = lo[i] < 0.0f ? q - ql : q + ql;
  }
  unsigned long long *o = sums + ((size_t)b * C + c) * K;
#pragma unroll
  for (int i = 0; i < P; ++i) {
    int k = j + LPC * i;
    if (k < K) o[k] = acc[i];
  }
}

// SCAN anchors, stage 2: exclusive prefix over chunks; the fixed-point phase is rounded to float.
// Block = SCAN_SEGS time segments x SCAN_KK partials (8 partials = one 64-byte run of the 64-bit sums per
// segment); each thread totals its segment, the segment totals are prefixed through shared memory, then each
// thread walks its segment again.  Many short segments keep every thread's serial walk to a few chunks and give
// enough blocks (ceil(K / 8) x B) to occupy the whole GPU.
constexpr int SCAN_KK = 8, SCAN_SEGS = 128;
__global__ void __launch_bounds__(SCAN_KK * SCAN_SEGS)
anchor_scan_kernel(const unsigned long long *__restrict__ sums, int B, int C, int K,
                   float *__restrict__ anchors, uint32_t *__restrict__ anchors_q) {
  __shared__ unsigned long long seg_tot[SCAN_SEGS][SCAN_KK + 1];
  const int kk = threadIdx.x % SCAN_KK, seg = threadIdx.x / SCAN_KK;
  const int k = blockIdx.x * SCAN_KK + kk, b = blockIdx.y;
  const bool ok = k < K;
  const int per = (C + SCAN_SEGS - 1) / SCAN_SEGS;
  const int c0 = min(C, seg * per), c1 = min(C, c0 + per);
  const unsigned long long *s = sums + (size_t)b * C * K + k;
  float *out = anchors + (size_t)b * C * K + k;
  uint32_t *outq = anchors_q ? anchors_q + (size_t)b * C * K + k : nullptr;
  unsigned long long tot = 0ull;
  if (ok)
    for (int c = c0; c < c1; ++c) tot += s[(size_t)c * K];
  seg_tot[seg][kk] = tot;
  __syncthreads();
  unsigned long long acc = 0ull;
  for (int s2 = 0; s2 < seg; ++s2) acc += seg_tot[s2][kk];
  if (!ok) return;
  for (int c = c0; c < c1; ++c) {
    float p = __ull2float_rn(acc) * 5.421010862427522e-20f;  // 2^-64
    out[(size_t)c * K] = p >= 1.0f ? 0.0f : p;
    if (outq) outq[(size_t)c * K] = (uint32_t)(acc >> 32);
    acc += s[(size_t)c * K];
  }
}

// FUNDAMENTAL anchors.  Every partial of a voice is a multiple of one fundamental, so one running sum per voice
// is enough: A[c] = sum_{n < 64 c} f0[n] / sr (mod 1) in Q0.64, and partial k starts chunk c at k * A[c] (mod 1),
// an exact integer product.  The per-frame quotient is taken to ~2^-48 (correctly rounded single-precision
// quotient plus the quotient of its exact remainder), so the sum over a whole render is good to ~2^-40 turns.
// What this mode leaves out, against the reference recurrence, is the rounding of every partial's own increment
// fl(fl(k f0) / sr) (the SCAN mode keeps it; both leave out the rounding of the phase add itself).
__device__ __forceinline__ unsigned long long inc_q64(float f0v, float sr, float rsr) {
  if (!(f0v >= 0.0f && f0v < sr)) {  // outside [0, sr): the fraction of f0 / sr; non-finite -> 0
    float r = f0v * rsr;
    r = r - floorf(r);
    if (!(r >= 0.0f && r < 1.0f)) r = 0.0f;
    return __float2ull_rn(r * 18446744073709551616.0f);
  }
  const float qh = div_by_const(f0v, sr, rsr);
  const float ql = __fmaf_rn(-qh, sr, f0v) * rsr;
  if (qh >= 1.0f) return 0ull;  // f0 within half an ulp of sr: one whole turn
  return __float2ull_rn(qh * 18446744073709551616.0f) + (unsigned long long)__float2ll_rn(ql * 18446744073709551616.0f);
}

// How many partials k = 1, 2, .. pass the Nyquist mask fl(k f0) < nyq of the reference (Examples/HarmonicE2E/
// Synth.swift:161-170): the products are monotone in k for f0 >= 0, so the passing partials are a prefix 1 .. kcut
// and one count per frame replaces a multiply and a compare per partial and frame.  Decided on the reference's own
// single-precision product, so a partial exactly at Nyquist flips exactly where the reference flips it.
__device__ __forceinline__ int nyquist_count(float f0v, float nyq, int K) {
  if (!(f0v == f0v)) return 0;            // NaN: every comparison is false
  if (!(f0v > 0.0f)) return K;            // zero or negative: every product is <= 0 < nyq
  const float r = nyq / f0v;
  if (!(r < (float)(K + 2))) return K;
  int k = (int)r + 1;
  if (k > K) k = K;
  while (k > 0 && !(__fmul_rn((float)k, f0v) < nyq)) --k;
  return k;
}

// One warp per (voice, chunk of 64 frames): the per-sample fundamental and output envelope of f0_track_kernel plus
// the chunk's total phase advance of the fundamental (Q0.64), and per frame the pair (phase advance of the
// fundamental from the chunk's first frame to this one: the wrapping sum of the frames' increments rounded to
// Q0.32; number of partials below Nyquist) that the render and its backward read instead of deriving them.
__global__ void __launch_bounds__(128)
f0_track_fund_kernel(const float2 *__restrict__ rowtab, const float *__restrict__ f0, int B, int T, int F, int K, float sr,
                     float rsr, float *__restrict__ f0t, const float *__restrict__ uv,
                     const float *__restrict__ gain, float scale, float *__restrict__ env,
                     unsigned long long *__restrict__ chunk_sum /* [B][C] */, int2 *__restrict__ trk /* [B][T] */) {
  const int C = (T + CH - 1) / CH;
  const int c = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31, b = blockIdx.y;
  if (c >= C) return;
  unsigned long long tot = 0ull;
  uint32_t carry = 0u;   // sum of the rounded increments of the chunk's frames before this half
#pragma unroll
  for (int h = 0; h < CH / 32; ++h) {
    const int n = c * CH + h * 32 + lane;
    uint32_t dq = 0u;
    int cnt = 0;
    if (n < T) {
      const float2 rt = rowtab[n];
      const int lo = __float_as_int(rt.x), hi = lo + 1 >= F ? 0 : lo + 1;
      const float fr = rt.y, omf = __fsub_rn(1.0f, fr);
      const float f0v = lerp_strict(omf, f0[(size_t)lo * B + b], fr, f0[(size_t)hi * B + b]);
      f0t[(size_t)b * T + n] = f0v;
      if (env) {
        const float gt = fmaf(fr, gain[(size_t)hi * B + b], omf * gain[(size_t)lo * B + b]);
        const float uvt = fmaf(fr, uv[(size_t)hi * B + b], omf * uv[(size_t)lo * B + b]);
        env[(size_t)b * T + n] = gt * uvt * scale;
      }
      const unsigned long long d64 = inc_q64(f0v, sr, rsr);
      tot += d64;
      dq = (uint32_t)((d64 + 0x80000000ull) >> 32);
      cnt = nyquist_count(f0v, sr * 0.5f, K);
    }
    if (trk) {   // warp-uniform
      uint32_t inc = dq;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += v;
      }
      if (n < T) trk[(size_t)b * T + n] = make_int2((int)(carry + inc - dq), cnt);
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, off);
  if (lane == 0) chunk_sum[(size_t)b * C + c] = tot;
}

// Exclusive prefix over the chunk totals of one voice (one block per voice, wrapping 64-bit adds = sums mod 1).
constexpr int FSCAN_THREADS = 1024;
__global__ void __launch_bounds__(FSCAN_THREADS)
fund_scan_kernel(const unsigned long long *__restrict__ chunk_sum, int C, unsigned long long *__restrict__ prefix) {
  __shared__ unsigned long long warp_tot[FSCAN_THREADS / 32];
  const unsigned long long *s = chunk_sum + (size_t)blockIdx.x * C;
  unsigned long long *o = prefix + (size_t)blockIdx.x * C;
  const int per = (C + FSCAN_THREADS - 1) / FSCAN_THREADS;
  const int c0 = min(C, (int)threadIdx.x * per), c1 = min(C, c0 + per);
  unsigned long long mine = 0ull;
  for (int c = c0; c < c1; ++c) mine += s[c];
  // inclusive scan of the thread totals: within the warp, then over the warp totals
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  unsigned long long inc = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const unsigned long long v = __shfl_up_sync(0xffffffffu, inc, off);
    if (lane >= off) inc += v;
  }
  if (lane == 31) warp_tot[w] = inc;
  __syncthreads();
  if (w == 0) {
    unsigned long long t = warp_tot[lane];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned long long v = __shfl_up_sync(0xffffffffu, t, off);
      if (lane >= off) t += v;
    }
    warp_tot[lane] = t;
  }
  __syncthreads();
  unsigned long long acc = inc - mine + (w > 0 ? warp_tot[w - 1] : 0ull);
  for (int c = c0; c < c1; ++c) {
    o[c] = acc;
    acc += s[c];
  }
}

// Render: a group of LPC lanes owns one (voice, chunk); lane j carries partials j, j+LPC, ...
// (P per lane) through the 64 frames; per frame the group reduces sum(sin*masked) and sum(masked)
// with shuffles; results of four frames are collected in lanes 0..3 and stored as one float4.
template <int LPC, int P>
__global__ void __launch_bounds__(128, 4)
harmonic_render_kernel(dgc_harmonic_params prm, float rsr, const float *__restrict__ play,
                       const float *__restrict__ f0, const float *__restrict__ uv,
                       const float *__restrict__ amps, const float *__restrict__ gain,
                       const float *__restrict__ anchors, float *__restrict__ audio) {
  constexpr int G = 128 / LPC;
  const int B = prm.B, T = prm.T, K = prm.K, F = prm.F;
  const int C = (T + CH - 1) / CH;
  const int g = threadIdx.x / LPC, j = threadIdx.x % LPC;
  int c = blockIdx.x * G + g;
  const int b = blockIdx.y;
  const bool active = c < C;
  if (!active) c = C - 1;
  const int n0 = c * CH;
  const float sr = prm.sample_rate, nyq = sr * 0.5f, kmax = (float)K, kf0 = (float)(j + 1);

  float ph[P], alo[P], ahi[P];
  const float *anc = anchors + ((size_t)b * C + c) * K;
#pragma unroll
  for (int i = 0; i < P; ++i) {
    int k = j + LPC * i;
    ph[i] = k < K ? anc[k] : 0.0f;
    alo[i] = 0.0f;
    ahi[i] = 0.0f;
  }
  int cur_lo = -1;
  float f0lo = 0, f0hi = 0, uvlo = 0, uvhi = 0, glo = 0, ghi = 0;
  float *dst = audio + (size_t)b * T;
  float keep = 0.0f;

#pragma unroll 1
  for (int s = 0; s < CH; ++s) {
    const int n = min(n0 + s, T - 1);
    int lo, hi;
    float fr;
    row_pos(play[n], F, lo, hi, fr);
    if (lo != cur_lo) {
      cur_lo = lo;
      const float *rl = amps + ((size_t)lo * B + b) * K, *rh = amps + ((size_t)hi * B + b) * K;
#pragma unroll
      for (int i = 0; i < P; ++i) {
        int k = j + LPC * i;
        alo[i] = k < K ? rl[k] : 0.0f;
        ahi[i] = k < K ? rh[k] : 0.0f;
      }
      f0lo = f0[(size_t)lo * B + b]; f0hi = f0[(size_t)hi * B + b];
      uvlo = uv[(size_t)lo * B + b]; uvhi = uv[(size_t)hi * B + b];
      glo = gain[(size_t)lo * B + b]; ghi = gain[(size_t)hi * B + b];
    }
    const float omf = __fsub_rn(1.0f, fr);
    const float f0t = lerp_strict(omf, f0lo, fr, f0hi);
    const float oa = omf;
    float s1 = 0.0f, s2 = 0.0f;
    // one decision per frame instead of one per partial: all increments of this frame in [0,1)?
    if (f0t >= 0.0f && __fmul_rn(kmax, f0t) < sr) {
#pragma unroll
      for (int i = 0; i < P; ++i) {
        float freq = __fmul_rn(partial_number(kf0, LPC * i), f0t);
        float a = fmaf(fr, ahi[i], oa * alo[i]);
        float m = freq < nyq ? a : 0.0f;
        s2 += m;
        s1 = fmaf(neg_sin_turns(ph[i]), -m, s1);
        float next = __fadd_rn(ph[i], div_by_const(freq, sr, rsr));
        ph[i] = next >= 1.0f ? __fadd_rn(next, -1.0f) : next;
      }
    } else {
#pragma unroll
      for (int i = 0; i < P; ++i) {
        float freq = __fmul_rn(partial_number(kf0, LPC * i), f0t);
        float a = fmaf(fr, ahi[i], oa * alo[i]);
        float m = freq < nyq ? a : 0.0f;
        s2 += m;
        s1 = fmaf(neg_sin_turns(ph[i]), -m, s1);
        ph[i] = phasor_step(ph[i], div_by_const(freq, sr, rsr));
      }
    }
#pragma unroll
    for (int off = LPC / 2; off > 0; off >>= 1) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, off);
      s2 += __shfl_xor_sync(0xffffffffu, s2, off);
    }
    const float gt = fmaf(fr, ghi, omf * glo), uvt = fmaf(fr, uvhi, omf * uvlo);
    const float val = s1 / (s2 + 1e-8f) * gt * uvt * prm.harmonic_scale;
    if (j == (s & 3)) keep = val;
    if ((s & 3) == 3) {
      // lanes 0..3 of the group hold frames s-3..s
      const int base = threadIdx.x - j;  // first lane of this group within the warp is (base & 31)
      float v1 = __shfl_sync(0xffffffffu, keep, (base & 31) + 1);
      float v2 = __shfl_sync(0xffffffffu, keep, (base & 31) + 2);
      float v3 = __shfl_sync(0xffffffffu, keep, (base & 31) + 3);
      if (active && j == 0) {
        int nn = n0 + s - 3;
        if (nn + 3 < T && ((((size_t)b * T + nn) & 3) == 0) && !prm.accumulate) {
          *reinterpret_cast<float4 *>(dst + nn) = make_float4(keep, v1, v2, v3);
        } else {
          float vv[4] = {keep, v1, v2, v3};
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (nn + u < T) dst[nn + u] = prm.accumulate ? dst[nn + u] + vv[u] : vv[u];
        }
      }
    }
  }
}

// Fundamental phase increment f0 / sr (mod 1) in Q0.32, to within one unit of 2^-32: the correctly rounded
// single-precision quotient plus the quotient of its exact remainder.
__device__ __forceinline__ uint32_t inc_q32(float f0v, float sr, float rsr) {
  if (!(f0v >= 0.0f && f0v < sr)) {  // outside [0, sr): the fraction of f0 / sr; non-finite -> 0
    float r = f0v * rsr;
    r = r - floorf(r);
    if (!(r >= 0.0f && r < 1.0f)) r = 0.0f;
    return __float2uint_rn(r * 4294967296.0f);
  }
  const float qh = div_by_const(f0v, sr, rsr);
  const float ql = __fmaf_rn(-qh, sr, f0v) * rsr;
  return __float2uint_rn(qh * 4294967296.0f) + (uint32_t)__float2int_rn(ql * 4294967296.0f);
}

// Sums of one 8-frame block held per lane (S1: sum of a sin, S2: sum of a, over the lane's partials) -> the lanes of
// the group are reduced so that lane (j & 7) ends with the totals of frame (j & 7), which it normalises, scales by
// the envelope and stores.  Lanes that differ in bits >= 3 of j hold disjoint partials of the same frames (plain
// butterfly); the low three bits go through a transposing butterfly (7 shuffles per quantity instead of 24).
template <int LPC, int MODE>
__device__ __forceinline__ void render_block_reduce_store(float (&S1)[8], float (&S2)[8], int j, int nb, int T, bool active,
                                                          const float *__restrict__ envp, const float *__restrict__ gp,
                                                          float *__restrict__ dst, int accumulate) {
  constexpr int FB = 8;
#pragma unroll
  for (int off = LPC / 2; off >= 8; off >>= 1) {
#pragma unroll
    for (int u = 0; u < FB; ++u) {
      S1[u] += __shfl_xor_sync(0xffffffffu, S1[u], off);
      S2[u] += __shfl_xor_sync(0xffffffffu, S2[u], off);
    }
  }
  const bool h2 = (j & 4) != 0, h1 = (j & 2) != 0, h0 = (j & 1) != 0;
  float A1[4], A2[4];
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const float k1 = h2 ? S1[v + 4] : S1[v], x1 = h2 ? S1[v] : S1[v + 4];
    const float k2 = h2 ? S2[v + 4] : S2[v], x2 = h2 ? S2[v] : S2[v + 4];
    A1[v] = k1 + __shfl_xor_sync(0xffffffffu, x1, 4);
    A2[v] = k2 + __shfl_xor_sync(0xffffffffu, x2, 4);
  }
  float B1[2], B2[2];
#pragma unroll
  for (int v = 0; v < 2; ++v) {
    const float k1 = h1 ? A1[v + 2] : A1[v], x1 = h1 ? A1[v] : A1[v + 2];
    const float k2 = h1 ? A2[v + 2] : A2[v], x2 = h1 ? A2[v] : A2[v + 2];
    B1[v] = k1 + __shfl_xor_sync(0xffffffffu, x1, 2);
    B2[v] = k2 + __shfl_xor_sync(0xffffffffu, x2, 2);
  }
  const float r1 = (h0 ? B1[1] : B1[0]) + __shfl_xor_sync(0xffffffffu, h0 ? B1[0] : B1[1], 1);
  const float r2 = (h0 ? B2[1] : B2[0]) + __shfl_xor_sync(0xffffffffu, h0 ? B2[0] : B2[1], 1);
  const int n = nb + (j & 7);
  if (active && j < 8 && n < T) {
    // the kernels take sin / cos of (2 pi p - pi): sin(2 pi p) = -sin(xr), cos(2 pi p) = -cos(xr)
    float val = -r1 / (r2 + 1e-8f) * envp[n];
    if (MODE == 1) val *= TWO_PI_F * gp[n];
    dst[n] = (MODE == 0 && accumulate) ? dst[n] + val : val;
  }
}

// SCAN-mode render with fixed-point phases.  The chunk anchors (exact sums of the reference's rounded
// single-precision increments, Q0.32) carry the long-term phase, so inside a 64-frame chunk the phase of
// partial k only has to advance by k * (f0 / sr): one integer add per partial and frame in Q0.32, wrapping
// for free.  Against the reference's float recurrence this drops the per-step rounding of the phase and
// of the increment inside one chunk (< 2e-6 turns), as the SCAN mode already does across chunks.
// The 23 top bits of the phase become the mantissa of a float in [1, 2) with one funnel shift, one FMA maps
// it to [-pi, pi) for the fast sine (sin(2 pi p - pi) = -sin(2 pi p); the sign is undone at the store).
// Same thread mapping as the float kernel; the sums of 8 frames are reduced over the group's lanes by a
// transposing butterfly (7 shuffles per quantity instead of 24), after which lane j owns frame j of the
// block, divides by the amplitude sum, applies the envelope and stores.
//
// MODE 0 renders audio.  MODE 1 writes, per frame, the phase gradient folded over the partials,
// sum_k k * dL/dphi_k[m] with dL/dphi_k = g_audio * env * a_k / (sum a + eps) * 2 pi cos(2 pi phi_k): the
// input of the temporal scan that gives dL/df0 (the same walk over the phases, cosine instead of sine).
template <int LPC, int P, int MODE>
__global__ void __launch_bounds__(128, 5)
harmonic_render_q_kernel(dgc_harmonic_params prm, float rsr, const float2 *__restrict__ rowtab,
                         const float *__restrict__ f0t, const float *__restrict__ env,
                         const float *__restrict__ amps, const uint32_t *__restrict__ anchors_q,
                         const unsigned long long *__restrict__ fund,
                         const float *__restrict__ g_audio, float *__restrict__ audio) {
  constexpr int G = 128 / LPC, FB = 8;
  constexpr float THREE_PI = 9.42477796076938f;
  const int B = prm.B, T = prm.T, K = prm.K, F = prm.F;
  const int C = (T + CH - 1) / CH;
  const int g = threadIdx.x / LPC, j = threadIdx.x % LPC;
  int c = blockIdx.x * G + g;
  const int b = blockIdx.y;
  const bool active = c < C;
  if (!active) c = C - 1;
  const int n0 = c * CH;
  const float sr = prm.sample_rate, nyq = sr * 0.5f, kf0 = (float)(j + 1);

  uint32_t q[P];
  float alo[P], dl[P];
  // chunk anchors: a table [B][C][K] (SCAN mode), or k times the fundamental's running sum (FUNDAMENTAL mode)
  const uint32_t *anc = anchors_q + ((size_t)b * C + c) * K;
  const unsigned long long fa = fund ? fund[(size_t)b * C + c] : 0ull;
#pragma unroll
  for (int i = 0; i < P; ++i) {
    int k = j + LPC * i;
    const uint32_t a0 = fund ? (uint32_t)(((unsigned long long)(k + 1) * fa) >> 32) : (k < K ? anc[k] : 0u);
    q[i] = a0 + 0x100u;  // + 2^8: dropping the low 9 bits below rounds to nearest
    alo[i] = 0.0f;
    dl[i] = 0.0f;
  }
  int cur_lo = -1;
  const float *f0p = f0t + (size_t)b * T, *envp = env + (size_t)b * T;
  float *dst = audio + (size_t)b * T;

#pragma unroll 1
  for (int blk = 0; blk < CH / FB; ++blk) {
    float S1[FB], S2[FB];
#pragma unroll
    for (int u = 0; u < FB; ++u) {
      const int n = min(n0 + blk * FB + u, T - 1);
      const float2 rt = rowtab[n];
      const int lo = __float_as_int(rt.x);
      const float fr = rt.y;
      if (lo != cur_lo) {
        cur_lo = lo;
        const int hi = lo + 1 >= F ? 0 : lo + 1;
        const float *rl = amps + ((size_t)lo * B + b) * K, *rh = amps + ((size_t)hi * B + b) * K;
#pragma unroll
        for (int i = 0; i < P; ++i) {
          int k = j + LPC * i;
          alo[i] = k < K ? rl[k] : 0.0f;
          dl[i] = k < K ? rh[k] - alo[i] : 0.0f;
        }
      }
      float s1 = 0.0f, s2 = 0.0f;
      {
        const float f0v = f0p[n];
        const uint32_t dq = inc_q32(f0v, sr, rsr);
        uint32_t incv = (uint32_t)(j + 1) * dq;
        const uint32_t step = (uint32_t)LPC * dq;
#pragma unroll
        for (int i = 0; i < P; ++i) {
          const float kf = partial_number(kf0, LPC * i);
          const float freq = __fmul_rn(kf, f0v);
          const float a = fmaf(fr, dl[i], alo[i]);
          const float ph1 = __uint_as_float(__funnelshift_r(q[i], 0x7Fu, 9));  // 1 + phase
          const float xr = fmaf(ph1, TWO_PI_F, -THREE_PI);
          if (freq < nyq) {  // Nyquist mask on the reference's single-precision product
            s2 += a;
            if (MODE == 0) s1 = fmaf(__sinf(xr), a, s1);
            else s1 = fmaf(__cosf(xr), kf * a, s1);
          }
          q[i] += incv;
          incv += step;
        }
      }
      S1[u] = s1;
      S2[u] = s2;
    }
    render_block_reduce_store<LPC, MODE>(S1, S2, j, n0 + blk * FB, T, active, envp,
                                         MODE == 1 ? g_audio + (size_t)b * T : nullptr, dst, prm.accumulate);
  }
}

// FUNDAMENTAL-mode render from the forward's tracks: ONE THREAD PER FRAME.
// The track kernel leaves, per voice and frame, the fundamental's phase advance inside its chunk (Q0.32) and the
// number of partials below Nyquist; with the chunk anchor A (Q0.64) the fundamental's phase at the frame is
// P = A + (advance << 32), and partial k has phase k P (mod 1): an exact integer product, built as a running 64-bit
// sum over k.  So a frame needs no state from other frames and no per-partial state at all, and a thread walks the
// partials of its own frame from 1 to the last audible one:
//   * nothing is reduced across lanes (the previous mapping spent a third of its instructions on the per-frame
//     butterfly and the per-lane bookkeeping around 13 partials);
//   * partials at or above Nyquist cost nothing, and since neighbouring frames have the same count (f0 moves
//     slowly) a warp's 32 loops end together;
//   * the amplitude rows are read straight from global memory: the 32 frames of a warp sit on the same control
//     row (or on two, across a row boundary), so every load is one broadcast line that stays in L1;
//   * ~40 registers per thread: the latencies of the dependent chain phase -> angle -> sine -> accumulate are
//     covered by resident warps.
// Per audible partial and frame: the 64-bit add, the shift, two multiply-adds, the sine, the two accumulates and
// a quarter of two 16-byte loads (VEC: K a multiple of 4 and 16-byte aligned rows; scalar loads otherwise).
template <bool VEC>
__global__ void __launch_bounds__(128)
harmonic_render_frame_kernel(dgc_harmonic_params prm, const float2 *__restrict__ rowtab, const float *__restrict__ env,
                             const float *__restrict__ amps, const unsigned long long *__restrict__ fund,
                             const int2 *__restrict__ trk, float2 *__restrict__ sums, float *__restrict__ audio) {
  constexpr float THREE_PI = 9.42477796076938f;
  const int B = prm.B, T = prm.T, K = prm.K, F = prm.F;
  const int C = (T + CH - 1) / CH;
  const int n = blockIdx.x * 128 + threadIdx.x, b = blockIdx.y;
  if (n >= T) return;
  const float2 rt = rowtab[n];
  const int lo = __float_as_int(rt.x), hi = lo + 1 >= F ? 0 : lo + 1;
  const float fr = rt.y;
  const int2 tk = trk[(size_t)b * T + n];
  const unsigned long long step = fund[(size_t)b * C + n / CH] + ((unsigned long long)(uint32_t)tk.x << 32);
  const int count = min(tk.y, K);
  const float *rl = amps + ((size_t)lo * B + b) * K, *rh = amps + ((size_t)hi * B + b) * K;
  // The two rows are used by 64 frames and then never again: every 128-byte line of them is a first touch from HBM
  // for the warp that walks into it.  The lanes of the warp ask for the lines the audible partials span up front
  // (lane l: line l of both rows), so the walk finds them on their way instead of stalling once per line.
  {
    const int l = threadIdx.x & 31, k0 = l * 32;
    if (k0 < count) {
      asm volatile("prefetch.global.L1 [%0];" ::"l"(rl + min(k0, K - 1)));
      asm volatile("prefetch.global.L1 [%0];" ::"l"(rh + min(k0, K - 1)));
    }
  }
  // k * P for k = 1, plus 2^8 in the high word for good: dropping the low 9 bits below then rounds to nearest
  unsigned long long acc = step + (0x100ull << 32);
  float s1 = 0.0f, s2 = 0.0f;
  auto partial = [&](float al, float ah) {
    const uint32_t q = (uint32_t)(acc >> 32);
    acc += step;
    const float a = fmaf(fr, ah - al, al);
    const float ph1 = __uint_as_float(__funnelshift_r(q, 0x7Fu, 9));  // 1 + phase
    const float xr = fmaf(ph1, TWO_PI_F, -THREE_PI);                  // 2 pi phase - pi
    s2 += a;
    s1 = fmaf(__sinf(xr), a, s1);
  };
  int k = 0;
  if (VEC) {
    // (keeping the next four partials' amplitudes in flight by hand, or staging the block's rows in shared memory,
    // both measured slower than this plain loop: 0.64 and 0.74 ms against 0.57 ms for the stage at 256 voices)
    const float4 *rl4 = reinterpret_cast<const float4 *>(rl), *rh4 = reinterpret_cast<const float4 *>(rh);
#pragma unroll 2
    for (; k + 4 <= count; k += 4) {
      const float4 l = __ldg(rl4 + (k >> 2)), h = __ldg(rh4 + (k >> 2));
      partial(l.x, h.x);
      partial(l.y, h.y);
      partial(l.z, h.z);
      partial(l.w, h.w);
    }
  } else {
#pragma unroll 4
    for (; k + 4 <= count; k += 4) {
      const float l0 = __ldg(rl + k), l1 = __ldg(rl + k + 1), l2 = __ldg(rl + k + 2), l3 = __ldg(rl + k + 3);
      const float h0 = __ldg(rh + k), h1 = __ldg(rh + k + 1), h2 = __ldg(rh + k + 2), h3 = __ldg(rh + k + 3);
      partial(l0, h0);
      partial(l1, h1);
      partial(l2, h2);
      partial(l3, h3);
    }
  }
  for (; k < count; ++k) partial(__ldg(rl + k), __ldg(rh + k));
  // sin(2 pi p) = -sin(2 pi p - pi)
  const float inv = 1.0f / (s2 + 1e-8f);
  const float ratio = -s1 * inv;
  if (sums) sums[(size_t)b * T + n] = make_float2(ratio, inv);   // for the backward: it then reduces nothing per frame
  const float val = ratio * env[(size_t)b * T + n];
  float *dst = audio + (size_t)b * T + n;
  *dst = prm.accumulate ? *dst + val : val;
}

template <int LPC, int P>
void launch_anchor_sum_t(dgc_ctx *ctx, int B, int T, int K, int C, const float *f0t, float sr, float rsr,
                         unsigned long long *sums) {
  constexpr int G = 128 / LPC;
  anchor_sum_kernel<LPC, P><<<dim3(dgc_div_up(C, G), B), 128, 0, ctx->stream>>>(f0t, B, T, K, sr, rsr, sums);
}

// lanes per (voice, chunk) group and partials per lane for K partials (K <= 512)
#define DGC_PICK_GROUP(K, CALL)            \
  do {                                     \
    if ((K) <= 8) CALL(8, 1);              \
    else if ((K) <= 16) CALL(8, 2);        \
    else if ((K) <= 32) CALL(8, 4);        \
    else if ((K) <= 64) CALL(8, 8);        \
    else if ((K) <= 104) CALL(8, 13);      \
    else if ((K) <= 112) CALL(16, 7);      \
    else if ((K) <= 128) CALL(16, 8);      \
    else if ((K) <= 256) CALL(32, 8);      \
    else CALL(32, 16);                     \
  } while (0)

void launch_anchor_sum(dgc_ctx *ctx, int B, int T, int K, int C, const float *f0t, float sr, float rsr,
                       unsigned long long *sums) {
#define CALL_SUM(LPC, P) launch_anchor_sum_t<LPC, P>(ctx, B, T, K, C, f0t, sr, rsr, sums)
  DGC_PICK_GROUP(K, CALL_SUM);
#undef CALL_SUM
}

template <int LPC, int P>
void launch_render(dgc_ctx *ctx, const dgc_harmonic_params &p, const float *play, const float *f0, const float *uv,
                   const float *amps, const float *gain, const float *anchors, float *audio) {
  int C = (p.T + CH - 1) / CH;
  constexpr int G = 128 / LPC;
  dim3 grid(dgc_div_up(C, G), p.B);
  harmonic_render_kernel<LPC, P><<<grid, 128, 0, ctx->stream>>>(p, 1.0f / p.sample_rate, play, f0, uv, amps, gain,
                                                                 anchors, audio);
}

template <int LPC, int P, int MODE>
void launch_render_q(dgc_ctx *ctx, const dgc_harmonic_params &p, const float2 *rowtab, const dgc_harmonic_extra &x,
                     const float *amps, const float *g_audio, float *out, bool keep_sums = false) {
  int C = (p.T + CH - 1) / CH;
  constexpr int G = 128 / LPC;
  dim3 grid(dgc_div_up(C, G), p.B);
  if (MODE == 0 && x.fund && x.trk) {
    const dim3 fgrid(dgc_div_up(p.T, 128), p.B);
    const bool vec = (p.K & 3) == 0 && (((uintptr_t)amps) & 15) == 0;
    float2 *keep = keep_sums ? x.sums : nullptr;
    if (vec) harmonic_render_frame_kernel<true><<<fgrid, 128, 0, ctx->stream>>>(p, rowtab, x.env, amps, x.fund, x.trk, keep, out);
    else harmonic_render_frame_kernel<false><<<fgrid, 128, 0, ctx->stream>>>(p, rowtab, x.env, amps, x.fund, x.trk, keep, out);
  } else
    harmonic_render_q_kernel<LPC, P, MODE><<<grid, 128, 0, ctx->stream>>>(p, 1.0f / p.sample_rate, rowtab, x.f0t, x.env,
                                                                           amps, x.anchors_q, x.fund, g_audio, out);
}

// The reverse scan of the reference's temporalGradScan (Sources/DGen/Emit+TemporalGradient.swift:54-88), per row e
// of T frames, walking n = T-1 .. 0 with carry = 0:
//     active = reset[n] > 0 ? 0 : carry ;  out[n] = scale * active ;  carry = g[n] + active
// i.e. out[n] = scale * sum of g[m] over n < m <= (the first frame after n with a reset, or T-1), and 0 on a reset
// frame itself: the gradient of the pre-update output still enters frame n even when reset[n] cuts the later
// recurrence.  reset is one signal [T] shared by all rows (the reference keeps one reset cell per frame); NULL =
// no resets, the plain exclusive suffix sum.
// One block per row; every thread owns a contiguous run of frames.  A run acts on the carry as c -> a c + b with
// a in {0, 1} (0 when the run holds a reset); those maps are composed over the later runs by a Hillis-Steele scan
// in double, then every thread walks its run from its incoming carry.
constexpr int TSCAN_THREADS = 1024;
__global__ void __launch_bounds__(TSCAN_THREADS)
temporal_suffix_scan_kernel(const float *__restrict__ g, const float *__restrict__ reset, int T, float scale,
                            float *__restrict__ out) {
  __shared__ double tot[TSCAN_THREADS];
  __shared__ unsigned char pass[TSCAN_THREADS];   // a of the composed map
  const float *row = g + (size_t)blockIdx.x * T;
  float *orow = out + (size_t)blockIdx.x * T;
  const int per = (T + TSCAN_THREADS - 1) / TSCAN_THREADS;
  const int n0 = min(T, (int)threadIdx.x * per), n1 = min(T, n0 + per);
  double s = 0.0;
  unsigned char a = 1;
  for (int n = n1 - 1; n >= n0; --n) {
    const bool r = reset && reset[n] > 0.0f;
    s = (double)row[n] + (r ? 0.0 : s);
    if (r) a = 0;
  }
  tot[threadIdx.x] = s;
  pass[threadIdx.x] = a;
  __syncthreads();
  // inclusive composition over this run and all later ones (10 steps): F_i o (F_{i+1} o ...)
  for (int off = 1; off < TSCAN_THREADS; off <<= 1) {
    const bool has = threadIdx.x + off < TSCAN_THREADS;
    const double b_late = has ? tot[threadIdx.x + off] : 0.0;
    const unsigned char a_late = has ? pass[threadIdx.x + off] : 1;
    __syncthreads();
    if (has) {
      if (pass[threadIdx.x]) tot[threadIdx.x] += b_late;
      pass[threadIdx.x] = pass[threadIdx.x] & a_late;
    }
    __syncthreads();
  }
  double carry = threadIdx.x + 1 < TSCAN_THREADS ? tot[threadIdx.x + 1] : 0.0;  // everything after this run, from 0
  for (int n = n1 - 1; n >= n0; --n) {
    const bool r = reset && reset[n] > 0.0f;
    const double active = r ? 0.0 : carry;
    orow[n] = (float)(active * (double)scale);
    carry = (double)row[n] + active;
  }
}

// g_f0[r][b] = sum over the frames whose lerp touches control row r of weight * G[b][n]: (1 - fr) where r is
// the floor row, fr where r is the next row (Sources/DGen/Emit+RowSelection.swift:166-199 backward).
__global__ void f0_rows_grad_kernel(const float2 *__restrict__ rowtab, const int *__restrict__ ranges,
                                    const float *__restrict__ G, int F, int B, int T, float *__restrict__ g_f0) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= F * B) return;
  const int r = idx / B, b = idx - r * B;
  const float *Gb = G + (size_t)b * T;
  double acc = 0.0;
  for (int run = 0; run < 2; ++run) {
    const int s0 = ranges[r * 4 + 2 * run], s1 = ranges[r * 4 + 2 * run + 1];
    for (int n = s0; n < s1; ++n) acc += (double)__fsub_rn(1.0f, rowtab[n].y) * (double)Gb[n];
  }
  const int prev = (r + F - 1) % F;
  for (int run = 0; run < 2; ++run) {
    const int s0 = ranges[prev * 4 + 2 * run], s1 = ranges[prev * 4 + 2 * run + 1];
    for (int n = s0; n < s1; ++n) acc += (double)rowtab[n].y * (double)Gb[n];
  }
  g_f0[(size_t)r * B + b] = (float)acc;
}

}  // namespace

const float2 *dgc_ctx_row_table(dgc_ctx *ctx, int F, int T) {
  auto key = std::make_pair(F, T);
  auto it = ctx->row_tables.find(key);
  if (it != ctx->row_tables.end()) return it->second;
  const float *play = nullptr;
  if (dgc_playhead(ctx, F, T, &play) != DGC_OK) return nullptr;
  float2 *d = nullptr;
  if (cudaMalloc(&d, ((size_t)T + 1) * sizeof(float2)) != cudaSuccess) {
    dgc_fail(ctx, DGC_ERR_OOM, "row table allocation failed");
    return nullptr;
  }
  // entry T: "no wrap" = 0x7f7f7f7f, above every frame index
  if (cudaMemsetAsync(d + T, 0x7f, sizeof(float2), ctx->stream) != cudaSuccess) {
    cudaFree(d);
    dgc_fail(ctx, DGC_ERR_CUDA, "row table preset failed");
    return nullptr;
  }
  row_table_kernel<<<dgc_div_up(T, 256), 256, 0, ctx->stream>>>(play, T, F, d);
  ctx->launches++;
  if (dgc_check_launch(ctx, "row_table") != DGC_OK) {
    cudaFree(d);
    return nullptr;
  }
  ctx->row_tables[key] = d;
  return d;
}

DGC_EXPORT int32_t dgc_clock_accum(dgc_ctx *ctx, float incr, float mn, float mx, float state0, int32_t T,
                                   float *out_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, out_dev && T > 0, "null output or T <= 0");
  DGC_REQUIRE(ctx, mx > mn, "max must exceed min");
  clock_accum_kernel<<<1, 32, 0, ctx->stream>>>(incr, mn, mx, state0, T, out_dev, 0, 0.f, 0.f);
  DGC_LAUNCHED(ctx, "clock_accum");
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_playhead(dgc_ctx *ctx, int32_t F, int32_t T, const float **out_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, out_dev && F > 0 && T > 0, "bad arguments");
  auto key = std::make_pair((int)F, (int)T);
  auto it = ctx->playheads.find(key);
  if (it != ctx->playheads.end()) {
    *out_dev = it->second;
    return DGC_OK;
  }
  float *d = nullptr;
  DGC_CUDA(ctx, cudaMalloc(&d, (size_t)T * sizeof(float)));
  // Examples/HarmonicE2E/Synth.swift:57-70, all in Float
  float fmax = (float)(F > 1 ? F - 1 : 0);
  float denom = (float)(T > 1 ? T - 1 : 1);
  float step = fmax / denom;
  float hi = fmax - 1e-4f;
  if (hi < 0.f) hi = 0.f;
  if (fmax <= 0.f) {
    DGC_CUDA(ctx, cudaMemsetAsync(d, 0, (size_t)T * sizeof(float), ctx->stream));
  } else {
    clock_accum_kernel<<<1, 32, 0, ctx->stream>>>(step, 0.f, fmax, 0.f, T, d, 1, 0.f, hi);
    ctx->launches++;
    int32_t rc = dgc_check_launch(ctx, "playhead");
    if (rc != DGC_OK) {
      cudaFree(d);
      return rc;
    }
  }
  ctx->playheads[key] = d;
  *out_dev = d;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_osc_bank_const(dgc_ctx *ctx, const float *freq_dev, const float *amp_dev, int32_t K,
                                      int32_t T, float sr, int32_t phase_mode, float *audio_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, freq_dev && amp_dev && audio_dev, "null pointer");
  DGC_REQUIRE(ctx, K > 0 && K <= 4096 && T > 0 && sr > 0, "size out of range");
  if (phase_mode == DGC_PHASE_DETERMINISTIC) {
    osc_const_det_kernel<<<dgc_div_up(T, 256), 256, 2 * K * sizeof(float), ctx->stream>>>(freq_dev, amp_dev, K, T, sr,
                                                                                          audio_dev);
    DGC_LAUNCHED(ctx, "osc_const_det");
    return DGC_OK;
  }
  if (phase_mode != DGC_PHASE_SEQUENTIAL)
    return dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "osc_bank_const: phase mode %d", phase_mode);
  int C = dgc_div_up(T, CH);
  float *anchors = dgc_ctx_scratch(ctx, (uint64_t)C * K);
  if (!anchors) return DGC_ERR_OOM;
  osc_const_anchor_seq_kernel<<<dgc_div_up(K, 32), 32, 0, ctx->stream>>>(freq_dev, K, T, sr, anchors);
  DGC_LAUNCHED(ctx, "osc_const_anchor_seq");
  osc_const_render_kernel<<<dgc_div_up(C, 4), 128, 0, ctx->stream>>>(freq_dev, amp_dev, anchors, K, T, sr, audio_dev);
  DGC_LAUNCHED(ctx, "osc_const_render");
  return DGC_OK;
}

DGC_EXPORT uint64_t dgc_harmonic_scratch_floats(const dgc_harmonic_params *p) {
  if (!p || p->B <= 0 || p->T <= 0 || p->K <= 0) return 0;
  uint64_t C = (uint64_t)(p->T + CH - 1) / CH;
  uint64_t lanes = (uint64_t)p->B * C * p->K;
  // f0 track [B][T] (rounded up to 4), anchors [B][C][K], chunk sums as 64-bit words (at least the 2 x [B][C]
  // words of the FUNDAMENTAL mode), output envelope [B][T], anchors as Q0.32 words
  const uint64_t sum_words = lanes > 2 * (uint64_t)p->B * C ? lanes : 2 * (uint64_t)p->B * C;
  // (+ the per-frame (phase advance, Nyquist count) pairs of the FUNDAMENTAL mode, [B][T] int2, and the per-frame
  // (normalised sum, reciprocal amplitude sum) pairs the forward leaves for its backward, [B][T] float2)
  return 2 * (((uint64_t)p->B * p->T + 3) & ~3ull) + lanes + 2 * sum_words + lanes + 16 +
         4 * (((uint64_t)p->B * p->T + 3) & ~3ull);
}

int32_t dgc_harmonic_prepare(dgc_ctx *ctx, const dgc_harmonic_params *p, const float *f0_dev, float *scratch,
                             const float **play_out, const float **anchors_out, const float *uv_dev,
                             const float *gain_dev, dgc_harmonic_extra *extra, bool already_prepared) {
  DGC_REQUIRE(ctx, p->B > 0 && p->T > 0 && p->F > 0 && p->K > 0 && p->K <= 512, "size out of range (K <= 512)");
  DGC_REQUIRE(ctx, p->B <= 65535, "B must be <= 65535");
  DGC_REQUIRE(ctx, p->sample_rate > 0, "sample rate must be positive");
  DGC_REQUIRE(ctx, p->phase_mode == DGC_PHASE_SEQUENTIAL || p->phase_mode == DGC_PHASE_SCAN ||
                       p->phase_mode == DGC_PHASE_FUNDAMENTAL, "phase mode");
  DGC_REQUIRE(ctx, (((uintptr_t)scratch) & 15) == 0, "scratch must be 16-byte aligned");
  const int B = p->B, T = p->T, K = p->K, F = p->F;
  const int C = dgc_div_up(T, CH);
  const float *play = nullptr;
  int32_t rc = dgc_playhead(ctx, F, T, &play);
  if (rc != DGC_OK) return rc;
  float *f0t = scratch;
  float *anchors = scratch + (((uint64_t)B * T + 3) & ~3ull);
  uint64_t lanes = (uint64_t)B * C * K;
  unsigned long long *sums = reinterpret_cast<unsigned long long *>(anchors + ((lanes + 1) & ~1ull));
  const uint64_t sum_words = lanes > 2 * (uint64_t)B * C ? lanes : 2 * (uint64_t)B * C;
  float *env = reinterpret_cast<float *>(sums + sum_words);
  uint32_t *anchors_q = reinterpret_cast<uint32_t *>(env + (((uint64_t)B * T + 3) & ~3ull));
  int2 *trk = reinterpret_cast<int2 *>(anchors_q + ((lanes + 3) & ~3ull));   // 8-byte aligned: every part before it is a multiple of 4 floats from a 16-byte aligned base
  const bool want_env = uv_dev && gain_dev && extra;
  const float2 *rowtab = dgc_ctx_row_table(ctx, F, T);
  if (!rowtab) return DGC_ERR_CUDA;
  const float sr = p->sample_rate, rsr = 1.0f / sr;
  // FUNDAMENTAL mode keeps two small arrays in the chunk-sum area: per-chunk totals [B][C], their prefix [B][C]
  unsigned long long *fund_sum = sums, *fund_prefix = sums + (uint64_t)B * C;
  if (already_prepared) {
    // nothing to launch
  } else if (p->phase_mode == DGC_PHASE_FUNDAMENTAL) {
    f0_track_fund_kernel<<<dim3(dgc_div_up(C, 4), B), 128, 0, ctx->stream>>>(rowtab, f0_dev, B, T, F, K, sr, rsr, f0t, uv_dev,
                                                                          gain_dev, p->harmonic_scale,
                                                                          want_env ? env : nullptr, fund_sum, trk);
    DGC_LAUNCHED(ctx, "f0_track_fund");
    fund_scan_kernel<<<B, FSCAN_THREADS, 0, ctx->stream>>>(fund_sum, C, fund_prefix);
    DGC_LAUNCHED(ctx, "fund_scan");
  } else {
  f0_track_kernel<<<dim3(dgc_div_up(T, 256), B), 256, 0, ctx->stream>>>(rowtab, f0_dev, B, T, F, f0t, uv_dev, gain_dev,
                                                                         p->harmonic_scale, want_env ? env : nullptr);
  DGC_LAUNCHED(ctx, "f0_track");
  if (p->phase_mode == DGC_PHASE_SEQUENTIAL) {
    anchor_seq_kernel<<<dgc_div_up(B * K, 32), 32, 0, ctx->stream>>>(f0t, B, T, K, sr, rsr, anchors);
    DGC_LAUNCHED(ctx, "anchor_seq");
  } else {
    launch_anchor_sum(ctx, B, T, K, C, f0t, sr, rsr, sums);
    DGC_LAUNCHED(ctx, "anchor_sum");
    anchor_scan_kernel<<<dim3(dgc_div_up(K, SCAN_KK), B), SCAN_KK * SCAN_SEGS, 0, ctx->stream>>>(sums, B, C, K, anchors,
                                                                             extra ? anchors_q : nullptr);
    DGC_LAUNCHED(ctx, "anchor_scan");
  }
  }
  if (extra) {
    extra->f0t = f0t;
    extra->env = want_env ? env : nullptr;
    extra->anchors_q = p->phase_mode == DGC_PHASE_SCAN ? anchors_q : nullptr;
    extra->fund = p->phase_mode == DGC_PHASE_FUNDAMENTAL ? fund_prefix : nullptr;
    extra->trk = p->phase_mode == DGC_PHASE_FUNDAMENTAL ? trk : nullptr;
    extra->sums = p->phase_mode == DGC_PHASE_FUNDAMENTAL
                      ? reinterpret_cast<float2 *>(trk + (((uint64_t)B * T + 3) & ~3ull)) : nullptr;
  }
  *play_out = play;
  *anchors_out = anchors;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_harmonic_render(dgc_ctx *ctx, const dgc_harmonic_params *p, const float *f0_dev,
                                       const float *uv_dev, const float *amps_dev, const float *gain_dev,
                                       float *scratch_dev, float *audio_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, p && f0_dev && uv_dev && amps_dev && gain_dev && audio_dev, "null pointer");
  float *scratch = scratch_dev ? scratch_dev : dgc_ctx_scratch(ctx, dgc_harmonic_scratch_floats(p));
  if (!scratch) return DGC_ERR_OOM;
  const float *play = nullptr, *anchors = nullptr;
  dgc_harmonic_extra extra;
  int32_t rc = dgc_harmonic_prepare(ctx, p, f0_dev, scratch, &play, &anchors, uv_dev, gain_dev, &extra);
  if (rc != DGC_OK) return rc;
  const int K = p->K;
  if (p->phase_mode == DGC_PHASE_SCAN || p->phase_mode == DGC_PHASE_FUNDAMENTAL) {
    DGC_REQUIRE(ctx, extra.env, "internal: the fixed-point render needs the envelope track");
    const float2 *rowtab = dgc_ctx_row_table(ctx, p->F, p->T);
    if (!rowtab) return DGC_ERR_CUDA;
    // a caller that hands in the scratch keeps it for the backward: leave the per-frame sums there
#define RENDERQ(LPC, P) launch_render_q<LPC, P, 0>(ctx, *p, rowtab, extra, amps_dev, nullptr, audio_dev, scratch_dev != nullptr)
    DGC_PICK_GROUP(K, RENDERQ);
#undef RENDERQ
  } else {
#define RENDER(LPC, P) launch_render<LPC, P>(ctx, *p, play, f0_dev, uv_dev, amps_dev, gain_dev, anchors, audio_dev)
    DGC_PICK_GROUP(K, RENDER);
#undef RENDER
  }
  DGC_LAUNCHED(ctx, "harmonic_render");
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_temporal_grad_scan(dgc_ctx *ctx, const float *g_dev, const float *reset_dev, int32_t E, int32_t T,
                                          float scale, float *out_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, g_dev && out_dev, "null pointer");
  DGC_REQUIRE(ctx, E > 0 && T > 0, "E and T must be positive");
  DGC_REQUIRE(ctx, g_dev != out_dev, "the scan is not in place");
  temporal_suffix_scan_kernel<<<E, TSCAN_THREADS, 0, ctx->stream>>>(g_dev, reset_dev, T, scale, out_dev);
  DGC_LAUNCHED(ctx, "temporal_grad_scan");
  return DGC_OK;
}

DGC_EXPORT uint64_t dgc_harmonic_f0_bwd_scratch_floats(const dgc_harmonic_params *p) {
  if (!p || p->B <= 0 || p->T <= 0 || p->K <= 0) return 0;
  return dgc_harmonic_scratch_floats(p) + 2 * (((uint64_t)p->B * p->T + 3) & ~3ull) + 16;
}

DGC_EXPORT int32_t dgc_harmonic_f0_bwd(dgc_ctx *ctx, const dgc_harmonic_params *p, const float *f0_dev,
                                       const float *uv_dev, const float *amps_dev, const float *gain_dev,
                                       const float *g_audio_dev, float *scratch_dev, float *g_f0_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, p && f0_dev && uv_dev && amps_dev && gain_dev && g_audio_dev && g_f0_dev, "null pointer");
  float *scratch = scratch_dev ? scratch_dev : dgc_ctx_scratch(ctx, dgc_harmonic_f0_bwd_scratch_floats(p));
  if (!scratch) return DGC_ERR_OOM;
  // the gradient walks the phases of the scan mode whatever mode rendered the audio: the two differ by
  // < 3e-5 turns, far inside the gradient tolerance
  dgc_harmonic_params q = *p;
  q.phase_mode = DGC_PHASE_SCAN;
  q.accumulate = 0;
  const float *play = nullptr, *anchors = nullptr;
  dgc_harmonic_extra extra;
  int32_t rc = dgc_harmonic_prepare(ctx, &q, f0_dev, scratch, &play, &anchors, uv_dev, gain_dev, &extra);
  if (rc != DGC_OK) return rc;
  const float2 *rowtab = dgc_ctx_row_table(ctx, q.F, q.T);
  const int *ranges = dgc_ctx_row_ranges(ctx, q.F, q.T);
  if (!rowtab || !ranges) return DGC_ERR_UNSUPPORTED;
  const uint64_t bt = ((uint64_t)q.B * q.T + 3) & ~3ull;
  float *gphi = scratch + ((dgc_harmonic_scratch_floats(&q) + 3) & ~3ull), *gsum = gphi + bt;
  const int K = q.K;
#define PHGRAD(LPC, P) launch_render_q<LPC, P, 1>(ctx, q, rowtab, extra, amps_dev, g_audio_dev, gphi)
  DGC_PICK_GROUP(K, PHGRAD);
#undef PHGRAD
  DGC_LAUNCHED(ctx, "harmonic_phase_grad");
  temporal_suffix_scan_kernel<<<q.B, TSCAN_THREADS, 0, ctx->stream>>>(gphi, nullptr, q.T, 1.0f / q.sample_rate, gsum);
  DGC_LAUNCHED(ctx, "temporal_grad_scan");
  f0_rows_grad_kernel<<<dgc_div_up((int64_t)q.F * q.B, 128), 128, 0, ctx->stream>>>(rowtab, ranges, gsum, q.F, q.B, q.T,
                                                                                g_f0_dev);
  DGC_LAUNCHED(ctx, "f0_rows_grad");
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_ctx_prepare_tables(dgc_ctx *ctx, int32_t F, int32_t T) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, F > 0 && T > 0, "F and T must be positive");
  if (!dgc_ctx_row_table(ctx, F, T)) return DGC_ERR_CUDA;      // builds the playhead as well
  dgc_ctx_row_ranges(ctx, F, T);   // only the backward kernels need the ranges: a clock they cannot handle is
                                   // reported by them, not here
  DGC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return DGC_OK;
}
