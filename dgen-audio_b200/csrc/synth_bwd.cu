// Backward of the batched harmonic+noise synthesis with respect to the controller outputs, and the
// controller's output heads.
//
// In the reference the gradient of the loss reaches the control tables through sampleRow's backward
// (frame-indexed scratch of the floor/ceil rows, Sources/DGen/Emit+RowSelection.swift:215-330) and is
// then summed over frames by tensorAccumulate (Sources/DGen/Emit+State.swift:50-115).  Which frames
// read a control row is a static property of the control clock, so here one thread group owns one
// (voice, control row): it walks exactly the frames whose floor row is r, accumulates the (1-frac)- and
// frac-weighted sums in registers, and row r's gradient is  floor_part[r] + ceil_part[r-1].  No
// atomics, fixed summation order.
#include "osc_common.cuh"

namespace {

using namespace dgosc;

// ---------------------------------------------------------------------------------------------
// heads: z [M][K+NB] -> amps = softplus(z[:K]) / (sum + 1e-6)   (Examples/HarmonicE2E/Model.swift:102-106)
//                        bands = sigmoid(z[K:])                   (band magnitudes in [0,1])
// one warp per row
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

__global__ void heads_fwd_kernel(const float *__restrict__ z, int M, int K, int NB, float *__restrict__ amps,
                                 float *__restrict__ bands) {
  int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= M) return;
  const float *zr = z + (size_t)row * (K + NB);
  float s = 0.0f;
  for (int k = lane; k < K; k += 32) s += softplus(zr[k]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  const float inv = 1.0f / (s + 1e-6f);
  for (int k = lane; k < K; k += 32) amps[(size_t)row * K + k] = softplus(zr[k]) * inv;
  for (int j = lane; j < NB; j += 32) bands[(size_t)row * NB + j] = sigmoid(zr[K + j]);
}

// amps_k = p_k / D, D = sum p + eps  =>  dL/dp_k = (g_k - sum_j g_j amps_j) / D ; dp/dz = sigmoid(z)
__global__ void heads_bwd_kernel(const float *__restrict__ z, const float *__restrict__ g_amps,
                                 const float *__restrict__ g_bands, int M, int K, int NB, float *__restrict__ gz) {
  int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= M) return;
  const float *zr = z + (size_t)row * (K + NB);
  const float *ga = g_amps + (size_t)row * K;
  float s = 0.0f, dot = 0.0f;
  for (int k = lane; k < K; k += 32) {
    float p = softplus(zr[k]);
    s += p;
    dot = fmaf(ga[k], p, dot);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, off);
    dot += __shfl_xor_sync(0xffffffffu, dot, off);
  }
  const float inv = 1.0f / (s + 1e-6f);
  const float mean = dot * inv;  // sum_j g_j amps_j
  float *o = gz + (size_t)row * (K + NB);
  for (int k = lane; k < K; k += 32) o[k] = (ga[k] - mean) * inv * sigmoid(zr[k]);
  for (int j = lane; j < NB; j += 32) {
    float sg = sigmoid(zr[K + j]);
    o[K + j] = g_bands[(size_t)row * NB + j] * sg * (1.0f - sg);
  }
}

// ---------------------------------------------------------------------------------------------
// noise FIR backward: gradient w.r.t. the tap table
//   y[n] = (sum_i x[n-NT+1+i] * ((1-fr) T[lo][i] + fr T[hi][i])) * ng[n] * scale
//   part_lo[b][r][i] = sum_{n: lo=r} (1-fr) g'[n] x[n-NT+1+i],  part_hi likewise with fr,  g' = g * ng * scale
// block = (row r, voice b); thread = tap i
// ---------------------------------------------------------------------------------------------
constexpr int FB_MAXRUN = 512;  // frames per control row the shared staging can hold

// A thread owns FOUR consecutive taps and walks the frames of the run four at a time: the two weights of a frame are
// broadcast loads shared by its eight multiply-adds, the signal window slides through registers (one 16-byte load
// of new samples per four frames), so four frames x four taps x two rows = 32 multiply-adds cost three 16-byte
// shared loads (one tap per thread: three 4-byte loads per two multiply-adds, and the 257th tap ran a pass of its
// own for a single thread).  Per tap the frames are summed in the same ascending order as before.
__global__ void __launch_bounds__(256)
fir_bwd_kernel(dgc_fir_params prm, const float *__restrict__ play, const int *__restrict__ ranges,
               const float *__restrict__ noise, const float *__restrict__ ngain, const float *__restrict__ g_audio,
               float *__restrict__ part_lo, float *__restrict__ part_hi, int32_t *status) {
  extern __shared__ __align__(16) float sh[];
  const int B = prm.B, T = prm.T, F = prm.F, NT = prm.taps;
  const int r = blockIdx.x, b = blockIdx.y, nth = blockDim.x;
  float *wl = sh, *wh = sh + FB_MAXRUN, *xs = sh + 2 * FB_MAXRUN;  // xs: FB_MAXRUN + NT + 11 (zero-extended)
  const float *xn = noise + (size_t)b * T, *g = g_audio + (size_t)b * T;
  const int i0 = 4 * threadIdx.x;          // taps i0 .. i0 + 3
  float acc_lo[4] = {0, 0, 0, 0}, acc_hi[4] = {0, 0, 0, 0};
  const int hi_row = r + 1 >= F ? 0 : r + 1;
  for (int run = 0; run < 2; ++run) {
    const int s0 = ranges[r * 4 + 2 * run], s1 = ranges[r * 4 + 2 * run + 1];
    const int len = s1 - s0;
    if (len <= 0) continue;
    if (len > FB_MAXRUN) {
      if (threadIdx.x == 0) atomicExch(status, 102);  // control rate too low for the staged run
      return;
    }
    const int len4 = (len + 3) & ~3;       // frames beyond the run carry zero weights
    __syncthreads();
    for (int i = threadIdx.x; i < len4; i += nth) {
      float vl = 0.0f, vh = 0.0f;
      if (i < len) {
        int n = s0 + i, lo, hi;
        float fr;
        row_pos(play[n], F, lo, hi, fr);
        float omf = 1.0f - fr;
        float ng = fmaf(fr, ngain[(size_t)hi_row * B + b], omf * ngain[(size_t)r * B + b]);
        float gp = g[n] * ng * prm.scale;
        vl = omf * gp;
        vh = fr * gp;
      }
      wl[i] = vl;
      wh[i] = vh;
    }
    const int xlen = len4 + 4 * nth + 8;   // every window a thread can read
    for (int i = threadIdx.x; i < xlen; i += nth) {
      int t = s0 - (NT - 1) + i;
      xs[i] = (i < len + NT - 1 && t >= 0 && t < T) ? xn[t] : 0.0f;
    }
    __syncthreads();
    if (i0 < NT) {
      const float4 *wl4 = reinterpret_cast<const float4 *>(wl), *wh4 = reinterpret_cast<const float4 *>(wh);
      const float4 *x4 = reinterpret_cast<const float4 *>(xs + i0);
      float xw[8];
      {
        const float4 v = x4[0];
        xw[0] = v.x; xw[1] = v.y; xw[2] = v.z; xw[3] = v.w;
      }
      for (int m4 = 0; m4 < len4 / 4; ++m4) {
        const float4 v = x4[m4 + 1], a4 = wl4[m4], c4 = wh4[m4];
        xw[4] = v.x; xw[5] = v.y; xw[6] = v.z; xw[7] = v.w;
        const float a[4] = {a4.x, a4.y, a4.z, a4.w}, c[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
        for (int s = 0; s < 4; ++s)       // frame m = 4 m4 + s: tap i0 + j reads xs[m + i0 + j]
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc_lo[j] = fmaf(a[s], xw[s + j], acc_lo[j]);
            acc_hi[j] = fmaf(c[s], xw[s + j], acc_hi[j]);
          }
#pragma unroll
        for (int j = 0; j < 4; ++j) xw[j] = xw[4 + j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = i0 + j;
    if (i >= NT) break;
    part_lo[((size_t)r * B + b) * NT + i] = acc_lo[j];
    part_hi[((size_t)r * B + b) * NT + i] = acc_hi[j];
  }
}

// the same four elements at a time (row_elems a multiple of 4, 16-byte aligned buffers); row_elems4 = row_elems / 4
__global__ void combine_rows4_kernel(const float4 *__restrict__ part_lo, const float4 *__restrict__ part_hi, int F,
                                     unsigned row_elems4, float4 *__restrict__ grad) {
  const unsigned e = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
  if (e >= row_elems4) return;
  const unsigned rp = r == 0 ? (unsigned)F - 1 : r - 1;
  const float4 a = part_lo[(size_t)r * row_elems4 + e], b = part_hi[(size_t)rp * row_elems4 + e];
  grad[(size_t)r * row_elems4 + e] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}

// grad[r] = part_lo[r] + part_hi[r-1]  (the ceil row of floor row F-1 is row 0)
__global__ void combine_rows_kernel(const float *__restrict__ part_lo, const float *__restrict__ part_hi, int F,
                                    size_t row_elems, float *__restrict__ grad) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)F * row_elems) return;
  size_t r = i / row_elems, e = i - r * row_elems;
  size_t rp = r == 0 ? (size_t)F - 1 : r - 1;
  grad[i] = part_lo[i] + part_hi[rp * row_elems + e];
}

// ---------------------------------------------------------------------------------------------
// harmonic bank backward: gradient w.r.t. the amplitude table amps [F][B][K]
//   audio[n] = S1/(S2+eps) * gu,  S1 = sum_k sin_k m_k,  S2 = sum_k m_k,  m_k = mask_k ((1-fr) A[lo][k] + fr A[hi][k])
//   d audio / d m_k = gu * (sin_k - S1/(S2+eps)) / (S2+eps)
// group of LPC lanes = one (voice, control row); phases are regenerated from the forward's anchors.
// ---------------------------------------------------------------------------------------------
template <int LPC, int P>
__global__ void __launch_bounds__(128)
harmonic_bwd_kernel(dgc_harmonic_params prm, float rsr, const float *__restrict__ play,
                    const int *__restrict__ ranges, const float *__restrict__ f0, const float *__restrict__ uv,
                    const float *__restrict__ amps, const float *__restrict__ gain,
                    const float *__restrict__ anchors, const float *__restrict__ g_audio,
                    float *__restrict__ part_lo, float *__restrict__ part_hi) {
  constexpr int G = 128 / LPC;
  const int B = prm.B, T = prm.T, K = prm.K, F = prm.F;
  const int C = (T + CH - 1) / CH;
  const int grp = threadIdx.x / LPC, j = threadIdx.x % LPC;
  int r = blockIdx.x * G + grp;
  const int b = blockIdx.y;
  const bool active = r < F;
  if (!active) r = F - 1;
  const int hi_row = r + 1 >= F ? 0 : r + 1;
  const float sr = prm.sample_rate, nyq = sr * 0.5f, kf0 = (float)(j + 1);
  float alo[P], ahi[P], pl[P], phh[P], ph[P];
  const float *rl = amps + ((size_t)r * B + b) * K, *rh = amps + ((size_t)hi_row * B + b) * K;
#pragma unroll
  for (int i = 0; i < P; ++i) {
    int k = j + LPC * i;
    alo[i] = k < K ? rl[k] : 0.0f;
    ahi[i] = k < K ? rh[k] : 0.0f;
    pl[i] = phh[i] = 0.0f;
    ph[i] = 0.0f;
  }
  const float f0lo = f0[(size_t)r * B + b], f0hi = f0[(size_t)hi_row * B + b];
  const float uvlo = uv[(size_t)r * B + b], uvhi = uv[(size_t)hi_row * B + b];
  const float glo = gain[(size_t)r * B + b], ghi = gain[(size_t)hi_row * B + b];
  const float *g = g_audio + (size_t)b * T;
  // the frames of a control row are contiguous runs; runs of different groups in a warp have different
  // lengths, so every group iterates to the longest run of the warp (shuffles need all lanes)
  for (int run = 0; run < 2; ++run) {
    const int s0 = ranges[r * 4 + 2 * run], s1 = ranges[r * 4 + 2 * run + 1];
    int len = active ? s1 - s0 : 0;
    int maxlen = len;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) maxlen = max(maxlen, __shfl_xor_sync(0xffffffffu, maxlen, off));
    if (maxlen <= 0) continue;
    // phases at s0: anchor of the chunk that contains s0, stepped to s0
    if (len > 0) {
      const int c0 = s0 / CH;
      const float *anc = anchors + ((size_t)b * C + c0) * K;
#pragma unroll
      for (int i = 0; i < P; ++i) {
        int k = j + LPC * i;
        ph[i] = k < K ? anc[k] : 0.0f;
      }
      for (int n = c0 * CH; n < s0; ++n) {
        int lo, hi;
        float fr;
        row_pos(play[n], F, lo, hi, fr);
        float omf = __fsub_rn(1.0f, fr);
        float f0t = lerp_strict(omf, f0[(size_t)lo * B + b], fr, f0[(size_t)hi * B + b]);
#pragma unroll
        for (int i = 0; i < P; ++i)
          ph[i] = phasor_step(ph[i], div_by_const(__fmul_rn(partial_number(kf0, LPC * i), f0t), sr, rsr));
      }
    }
    for (int m = 0; m < maxlen; ++m) {
      const bool live = m < len;
      const int n = live ? s0 + m : 0;
      if (live && (n % CH) == 0) {  // the forward re-anchors at every chunk boundary
        const float *anc = anchors + ((size_t)b * C + n / CH) * K;
#pragma unroll
        for (int i = 0; i < P; ++i) {
          int k = j + LPC * i;
          ph[i] = k < K ? anc[k] : 0.0f;
        }
      }
      int lo, hi;
      float fr;
      row_pos(play[n], F, lo, hi, fr);
      const float omf = __fsub_rn(1.0f, fr);
      const float f0t = lerp_strict(omf, f0lo, fr, f0hi);
      float sn[P], mk[P];
      float s1v = 0.0f, s2v = 0.0f;
#pragma unroll
      for (int i = 0; i < P; ++i) {
        float freq = __fmul_rn(partial_number(kf0, LPC * i), f0t);
        float a = fmaf(fr, ahi[i], omf * alo[i]);
        mk[i] = freq < nyq ? 1.0f : 0.0f;
        float mm = mk[i] * a;
        sn[i] = sin_turns(ph[i]);
        s2v += mm;
        s1v = fmaf(sn[i], mm, s1v);
        if (live) ph[i] = phasor_step(ph[i], div_by_const(freq, sr, rsr));
      }
#pragma unroll
      for (int off = LPC / 2; off > 0; off >>= 1) {
        s1v += __shfl_xor_sync(0xffffffffu, s1v, off);
        s2v += __shfl_xor_sync(0xffffffffu, s2v, off);
      }
      if (live) {
        const float gt = fmaf(fr, ghi, omf * glo), uvt = fmaf(fr, uvhi, omf * uvlo);
        const float inv = 1.0f / (s2v + 1e-8f);
        const float ratio = s1v * inv;
        const float c = g[n] * gt * uvt * prm.harmonic_scale * inv;
        const float cl = c * omf, chh = c * fr;
#pragma unroll
        for (int i = 0; i < P; ++i) {
          float d = (sn[i] - ratio) * mk[i];
          pl[i] = fmaf(cl, d, pl[i]);
          phh[i] = fmaf(chh, d, phh[i]);
        }
      }
    }
  }
  if (active) {
    float *ol = part_lo + ((size_t)r * B + b) * K, *oh = part_hi + ((size_t)r * B + b) * K;
#pragma unroll
    for (int i = 0; i < P; ++i) {
      int k = j + LPC * i;
      if (k < K) {
        ol[k] = pl[i];
        oh[k] = phh[i];
      }
    }
  }
}

// The same gradient with the fixed-point phases of the scan-mode render (see harmonic_render_q_kernel in
// osc_bank.cu): phases in Q0.32 from the Q0.32 chunk anchors, advanced by k * (f0 / sr) per frame with one
// integer add; the per-sample fundamental, the output envelope gain * uv * scale and the control-row
// position come from the precursor kernel's tracks instead of being re-derived per lane; the walk from a
// chunk anchor to the first frame of a run adds up the fundamental's increments once (shared by all
// partials, split over the group's lanes) instead of stepping every partial.
__device__ __forceinline__ uint32_t inc_q32_bwd(float f0v, float sr, float rsr) {
  if (!(f0v >= 0.0f && f0v < sr)) {
    float r = f0v * rsr;
    r = r - floorf(r);
    if (!(r >= 0.0f && r < 1.0f)) r = 0.0f;
    return __float2uint_rn(r * 4294967296.0f);
  }
  const float qh = div_by_const(f0v, sr, rsr);
  const float ql = __fmaf_rn(-qh, sr, f0v) * rsr;
  return __float2uint_rn(qh * 4294967296.0f) + (uint32_t)__float2int_rn(ql * 4294967296.0f);
}

//
// TRK (FUNDAMENTAL mode, tracks of the forward at hand): the fundamental's phase advance inside the chunk and the
// number of partials below Nyquist are read per frame from the forward's track; the phase of partial k is
// anchor_k + k * phi with phi that advance, so no per-partial state advances and both loops over this lane's partials end at the
// last audible one (the partials at or above Nyquist contribute an exact zero and are not visited).
// SUMS (with TRK): the forward left, per frame, the normalised sum and the reciprocal of the amplitude sum; the
// group then reduces nothing over its lanes -- per audible partial and frame the phase, the sine and the two
// gradient accumulates remain.
template <int LPC, int P, bool TRK, bool SUMS>
__global__ void __launch_bounds__(128)
harmonic_bwd_q_kernel(dgc_harmonic_params prm, float rsr, const float2 *__restrict__ rowtab,
                      const int *__restrict__ ranges, const float *__restrict__ f0t, const float *__restrict__ env,
                      const float *__restrict__ amps, const uint32_t *__restrict__ anchors_q,
                      const unsigned long long *__restrict__ fund, const int2 *__restrict__ trk,
                      const float2 *__restrict__ sums, const float *__restrict__ g_audio, float *__restrict__ part_lo,
                      float *__restrict__ part_hi) {
  constexpr int G = 128 / LPC;
  constexpr int LOG_LPC = LPC == 8 ? 3 : LPC == 16 ? 4 : 5;
  constexpr float THREE_PI = 9.42477796076938f;
  const int B = prm.B, T = prm.T, K = prm.K, F = prm.F;
  const int C = (T + CH - 1) / CH;
  const int grp = threadIdx.x / LPC, j = threadIdx.x % LPC;
  int r = blockIdx.x * G + grp;
  const int b = blockIdx.y;
  const bool active = r < F;
  if (!active) r = F - 1;
  const int hi_row = r + 1 >= F ? 0 : r + 1;
  const float sr = prm.sample_rate, nyq = sr * 0.5f, kf0 = (float)(j + 1);
  float alo[P], dl[P], pl[P], phh[P];
  uint32_t q[P];
  const float *rl = amps + ((size_t)r * B + b) * K, *rh = amps + ((size_t)hi_row * B + b) * K;
#pragma unroll
  for (int i = 0; i < P; ++i) {
    int k = j + LPC * i;
    alo[i] = k < K ? rl[k] : 0.0f;
    dl[i] = k < K ? rh[k] - alo[i] : 0.0f;
    pl[i] = phh[i] = 0.0f;
    q[i] = 0u;
  }
  const float *g = g_audio + (size_t)b * T, *f0p = f0t + (size_t)b * T, *envp = env + (size_t)b * T;
  const int2 *tkp = trk + (size_t)b * T;
  uint32_t phi = 0u;   // TRK: the fundamental's increments summed from the chunk start to the current frame
  for (int run = 0; run < 2; ++run) {
    const int s0 = ranges[r * 4 + 2 * run], s1 = ranges[r * 4 + 2 * run + 1];
    const int len = active ? s1 - s0 : 0;
    int maxlen = len;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) maxlen = max(maxlen, __shfl_xor_sync(0xffffffffu, maxlen, off));
    if (maxlen <= 0) continue;
    // phases at s0: chunk anchor + k * (sum of the fundamental's increments from the chunk start to s0);
    // the lanes of the group share the walk (every lane takes part in the shuffles, with 0 when it has no run)
    {
      const int c0 = len > 0 ? s0 / CH : 0;
      uint32_t part = 0u;
      if (len > 0)
        for (int n = c0 * CH + j; !TRK && n < s0; n += LPC) part += inc_q32_bwd(f0p[n], sr, rsr);
#pragma unroll
      for (int off = LPC / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
      if (len > 0) {
        // chunk anchors: the forward's table, or k times the fundamental's running sum (FUNDAMENTAL mode)
        const uint32_t *anc = anchors_q + ((size_t)b * C + c0) * K;
        const unsigned long long fa = fund ? fund[(size_t)b * C + c0] : 0ull;
#pragma unroll
        for (int i = 0; i < P; ++i) {
          int k = j + LPC * i;
          const uint32_t a0 = fund ? (uint32_t)(((unsigned long long)(k + 1) * fa) >> 32) : (k < K ? anc[k] : 0u);
          q[i] = a0 + 0x100u + (TRK ? 0u : (uint32_t)(k + 1) * part);
        }
        phi = part;
      }
    }
    for (int m = 0; m < maxlen; ++m) {
      const bool live = m < len;
      const int n = live ? s0 + m : 0;
      if (live && (n % CH) == 0) {  // the forward re-anchors at every chunk boundary
        const uint32_t *anc = anchors_q + ((size_t)b * C + n / CH) * K;
        const unsigned long long fa = fund ? fund[(size_t)b * C + n / CH] : 0ull;
#pragma unroll
        for (int i = 0; i < P; ++i) {
          int k = j + LPC * i;
          const uint32_t a0 = fund ? (uint32_t)(((unsigned long long)(k + 1) * fa) >> 32) : (k < K ? anc[k] : 0u);
          q[i] = a0 + 0x100u;
        }
        phi = 0u;
      }
      const float fr = rowtab[n].y, omf = __fsub_rn(1.0f, fr);
      if (TRK) {
        const int2 tk = tkp[n];
        phi = (uint32_t)tk.x;   // the fundamental's phase advance from the chunk's first frame, from the forward's track
        const int ilim = live ? max(tk.y - j + LPC - 1, 0) >> LOG_LPC : 0;   // partial j + LPC i + 1 <= count  <=>  i < ilim
        uint32_t w = (uint32_t)(j + 1) * phi;          // k * phi as a running sum over this lane's partials
        const uint32_t r = phi << LOG_LPC;
        if (SUMS) {
          if (live) {
            const float2 sm = sums[(size_t)b * T + n];   // (sum a sin / (sum a + eps), 1 / (sum a + eps)) of the forward
            const float c = g[n] * envp[n] * sm.y;
            const float cl = c * omf, chh = c * fr;
#pragma unroll
            for (int i = 0; i < P; ++i) {
              if (i >= ilim) break;
              const float ph1 = __uint_as_float(__funnelshift_r(q[i] + w, 0x7Fu, 9));
              w += r;
              const float d = -__sinf(fmaf(ph1, TWO_PI_F, -THREE_PI)) - sm.x;   // sin(2 pi p) - normalised sum
              pl[i] = fmaf(cl, d, pl[i]);
              phh[i] = fmaf(chh, d, phh[i]);
            }
          }
          continue;
        }
        float sn[P];
        float s1v = 0.0f, s2v = 0.0f;
#pragma unroll
        for (int i = 0; i < P; ++i) {
          if (i >= ilim) break;
          const uint32_t qq = q[i] + w;
          w += r;
          const float a = fmaf(fr, dl[i], alo[i]);
          const float ph1 = __uint_as_float(__funnelshift_r(qq, 0x7Fu, 9));
          sn[i] = -__sinf(fmaf(ph1, TWO_PI_F, -THREE_PI));   // sin(2 pi p)
          s2v += a;
          s1v = fmaf(sn[i], a, s1v);
        }
#pragma unroll
        for (int off = LPC / 2; off > 0; off >>= 1) {
          s1v += __shfl_xor_sync(0xffffffffu, s1v, off);
          s2v += __shfl_xor_sync(0xffffffffu, s2v, off);
        }
        if (live) {
          const float inv = 1.0f / (s2v + 1e-8f);
          const float ratio = s1v * inv;
          const float c = g[n] * envp[n] * inv;
          const float cl = c * omf, chh = c * fr;
#pragma unroll
          for (int i = 0; i < P; ++i) {
            if (i >= ilim) break;
            const float d = sn[i] - ratio;
            pl[i] = fmaf(cl, d, pl[i]);
            phh[i] = fmaf(chh, d, phh[i]);
          }
        }
        continue;
      }
      const float f0v = f0p[n];
      const uint32_t dq = inc_q32_bwd(f0v, sr, rsr);
      uint32_t incv = (uint32_t)(j + 1) * dq;
      const uint32_t step = (uint32_t)LPC * dq;
      float sn[P], mm[P];
      float s1v = 0.0f, s2v = 0.0f;
#pragma unroll
      for (int i = 0; i < P; ++i) {
        const float freq = __fmul_rn(partial_number(kf0, LPC * i), f0v);
        const float a = fmaf(fr, dl[i], alo[i]);
        const float ph1 = __uint_as_float(__funnelshift_r(q[i], 0x7Fu, 9));
        sn[i] = -__sinf(fmaf(ph1, TWO_PI_F, -THREE_PI));   // sin(2 pi p)
        mm[i] = freq < nyq ? 1.0f : 0.0f;
        const float am = mm[i] * a;
        s2v += am;
        s1v = fmaf(sn[i], am, s1v);
        if (live) q[i] += incv;
        incv += step;
      }
#pragma unroll
      for (int off = LPC / 2; off > 0; off >>= 1) {
        s1v += __shfl_xor_sync(0xffffffffu, s1v, off);
        s2v += __shfl_xor_sync(0xffffffffu, s2v, off);
      }
      if (live) {
        const float inv = 1.0f / (s2v + 1e-8f);
        const float ratio = s1v * inv;
        const float c = g[n] * envp[n] * inv;
        const float cl = c * omf, chh = c * fr;
#pragma unroll
        for (int i = 0; i < P; ++i) {
          const float d = (sn[i] - ratio) * mm[i];
          pl[i] = fmaf(cl, d, pl[i]);
          phh[i] = fmaf(chh, d, phh[i]);
        }
      }
    }
  }
  if (active) {
    float *ol = part_lo + ((size_t)r * B + b) * K, *oh = part_hi + ((size_t)r * B + b) * K;
#pragma unroll
    for (int i = 0; i < P; ++i) {
      int k = j + LPC * i;
      if (k < K) {
        ol[k] = pl[i];
        oh[k] = phh[i];
      }
    }
  }
}

// grad[r] = part_lo[r] + part_hi[r-1] over F rows of row_elems floats
void launch_combine_rows(dgc_ctx *ctx, const float *pl, const float *ph, int F, size_t row_elems, float *grad) {
  const bool vec = (row_elems & 3) == 0 && F <= 65535 &&
                   ((((uintptr_t)pl) | ((uintptr_t)ph) | ((uintptr_t)grad)) & 15) == 0;
  if (vec) {
    const unsigned re4 = (unsigned)(row_elems / 4);
    combine_rows4_kernel<<<dim3(dgc_div_up((int64_t)re4, 256), F), 256, 0, ctx->stream>>>(
        reinterpret_cast<const float4 *>(pl), reinterpret_cast<const float4 *>(ph), F, re4,
        reinterpret_cast<float4 *>(grad));
  } else {
    const size_t n = (size_t)F * row_elems;
    combine_rows_kernel<<<dgc_div_up((int64_t)n, 256), 256, 0, ctx->stream>>>(pl, ph, F, row_elems, grad);
  }
}

template <int LPC, int P>
void launch_hbwd_q(dgc_ctx *ctx, const dgc_harmonic_params &p, const float2 *rowtab, const int *ranges,
                   const dgc_harmonic_extra &x, const float *amps, const float *g_audio, float *pl, float *ph,
                   bool have_sums) {
  constexpr int G = 128 / LPC;
  const dim3 grid(dgc_div_up(p.F, G), p.B);
  if (x.fund && x.trk && have_sums && x.sums)
    harmonic_bwd_q_kernel<LPC, P, true, true><<<grid, 128, 0, ctx->stream>>>(
        p, 1.0f / p.sample_rate, rowtab, ranges, x.f0t, x.env, amps, x.anchors_q, x.fund, x.trk, x.sums, g_audio, pl, ph);
  else if (x.fund && x.trk)
    harmonic_bwd_q_kernel<LPC, P, true, false><<<grid, 128, 0, ctx->stream>>>(
        p, 1.0f / p.sample_rate, rowtab, ranges, x.f0t, x.env, amps, x.anchors_q, x.fund, x.trk, nullptr, g_audio, pl, ph);
  else
    harmonic_bwd_q_kernel<LPC, P, false, false><<<grid, 128, 0, ctx->stream>>>(
        p, 1.0f / p.sample_rate, rowtab, ranges, x.f0t, x.env, amps, x.anchors_q, x.fund, x.trk, nullptr, g_audio, pl, ph);
}

template <int LPC, int P>
void launch_hbwd(dgc_ctx *ctx, const dgc_harmonic_params &p, const float *play, const int *ranges, const float *f0,
                 const float *uv, const float *amps, const float *gain, const float *anchors, const float *g_audio,
                 float *pl, float *ph) {
  constexpr int G = 128 / LPC;
  harmonic_bwd_kernel<LPC, P><<<dim3(dgc_div_up(p.F, G), p.B), 128, 0, ctx->stream>>>(
      p, 1.0f / p.sample_rate, play, ranges, f0, uv, amps, gain, anchors, g_audio, pl, ph);
}

}  // namespace

DGC_EXPORT int32_t dgc_hn_heads_fwd(dgc_ctx *ctx, const float *z_dev, int32_t M, int32_t K, int32_t NB,
                                    float *amps_dev, float *bands_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, z_dev && amps_dev && bands_dev, "null pointer");
  DGC_REQUIRE(ctx, M > 0 && K > 0 && NB > 0, "size out of range");
  heads_fwd_kernel<<<dgc_div_up((int64_t)M * 32, 256), 256, 0, ctx->stream>>>(z_dev, M, K, NB, amps_dev, bands_dev);
  DGC_LAUNCHED(ctx, "heads_fwd");
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_hn_heads_bwd(dgc_ctx *ctx, const float *z_dev, const float *g_amps_dev,
                                    const float *g_bands_dev, int32_t M, int32_t K, int32_t NB, float *gz_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, z_dev && g_amps_dev && g_bands_dev && gz_dev, "null pointer");
  DGC_REQUIRE(ctx, M > 0 && K > 0 && NB > 0, "size out of range");
  heads_bwd_kernel<<<dgc_div_up((int64_t)M * 32, 256), 256, 0, ctx->stream>>>(z_dev, g_amps_dev, g_bands_dev, M, K,
                                                                             NB, gz_dev);
  DGC_LAUNCHED(ctx, "heads_bwd");
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_fir_noise_bwd(dgc_ctx *ctx, const dgc_fir_params *p, const float *noise_dev,
                                     const float *noise_gain_dev, const float *g_audio_dev, float *g_taps_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, p && noise_dev && noise_gain_dev && g_audio_dev && g_taps_dev, "null pointer");
  DGC_REQUIRE(ctx, p->B > 0 && p->B <= 65535 && p->T > 0 && p->F > 0, "size out of range");
  DGC_REQUIRE(ctx, p->taps >= 1 && p->taps <= 1024, "taps must be in 1..1024");
  const float *play = nullptr;
  int32_t rc = dgc_playhead(ctx, p->F, p->T, &play);
  if (rc != DGC_OK) return rc;
  const int *ranges = dgc_ctx_row_ranges(ctx, p->F, p->T);
  if (!ranges) return DGC_ERR_UNSUPPORTED;
  const size_t n = (size_t)p->F * p->B * p->taps;
  float *part = dgc_ctx_scratch(ctx, 2 * n + 8);
  if (!part) return DGC_ERR_OOM;
  // four taps per thread, whole warps
  const int nth = dgc_div_up(dgc_div_up(p->taps, 4), 32) * 32;
  size_t smem = (size_t)(3 * FB_MAXRUN + 4 * nth + 16) * sizeof(float);
  fir_bwd_kernel<<<dim3(p->F, p->B), nth, smem, ctx->stream>>>(*p, play, ranges, noise_dev, noise_gain_dev,
                                                                g_audio_dev, part, part + n, ctx->status_dev);
  DGC_LAUNCHED(ctx, "fir_bwd");
  launch_combine_rows(ctx, part, part + n, p->F, (size_t)p->B * p->taps, g_taps_dev);
  DGC_LAUNCHED(ctx, "combine_rows");
  return DGC_OK;
}

DGC_EXPORT uint64_t dgc_harmonic_bwd_scratch_floats(const dgc_harmonic_params *p) {
  if (!p || p->B <= 0 || p->T <= 0 || p->K <= 0 || p->F <= 0) return 0;
  return dgc_harmonic_scratch_floats(p) + 2ull * p->F * p->B * p->K + 16;
}

static int32_t harmonic_render_bwd_impl(dgc_ctx *ctx, const dgc_harmonic_params *p, const float *f0_dev,
                                        const float *uv_dev, const float *amps_dev, const float *gain_dev,
                                        const float *g_audio_dev, float *scratch_dev, float *g_amps_dev,
                                        bool prepared) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, p && f0_dev && uv_dev && amps_dev && gain_dev && g_audio_dev && g_amps_dev, "null pointer");
  DGC_REQUIRE(ctx, !prepared || scratch_dev, "the prepared variant needs the forward call's scratch");
  float *scratch = scratch_dev ? scratch_dev : dgc_ctx_scratch(ctx, dgc_harmonic_bwd_scratch_floats(p));
  if (!scratch) return DGC_ERR_OOM;
  const float *play = nullptr, *anchors = nullptr;
  dgc_harmonic_extra extra;
  int32_t rc = dgc_harmonic_prepare(ctx, p, f0_dev, scratch, &play, &anchors, uv_dev, gain_dev, &extra, prepared);
  if (rc != DGC_OK) return rc;
  const int *ranges = dgc_ctx_row_ranges(ctx, p->F, p->T);
  if (!ranges) return DGC_ERR_UNSUPPORTED;
  const size_t n = (size_t)p->F * p->B * p->K;
  float *pl = scratch + ((dgc_harmonic_scratch_floats(p) + 3) & ~3ull), *ph = pl + n;
  const int K = p->K;
  const bool fixed_point = extra.env && ((p->phase_mode == DGC_PHASE_SCAN && extra.anchors_q) ||
                                         (p->phase_mode == DGC_PHASE_FUNDAMENTAL && extra.fund));
  DGC_REQUIRE(ctx, fixed_point || p->phase_mode != DGC_PHASE_FUNDAMENTAL, "internal: fundamental mode without its tracks");
  const float2 *rowtab = fixed_point ? dgc_ctx_row_table(ctx, p->F, p->T) : nullptr;
  if (fixed_point && !rowtab) return DGC_ERR_CUDA;
#define HBWD(LPC, P)                                                                                                  \
  do {                                                                                                                \
    if (fixed_point) launch_hbwd_q<LPC, P>(ctx, *p, rowtab, ranges, extra, amps_dev, g_audio_dev, pl, ph, prepared);  \
    else launch_hbwd<LPC, P>(ctx, *p, play, ranges, f0_dev, uv_dev, amps_dev, gain_dev, anchors, g_audio_dev, pl, ph); \
  } while (0)
  if (K <= 8) HBWD(8, 1);
  else if (K <= 16) HBWD(8, 2);
  else if (K <= 32) HBWD(8, 4);
  else if (K <= 64) HBWD(8, 8);
  else if (K <= 112) HBWD(16, 7);
  else if (K <= 128) HBWD(16, 8);
  else if (K <= 256) HBWD(32, 8);
  else HBWD(32, 16);
#undef HBWD
  DGC_LAUNCHED(ctx, "harmonic_bwd");
  launch_combine_rows(ctx, pl, ph, p->F, (size_t)p->B * K, g_amps_dev);
  DGC_LAUNCHED(ctx, "combine_rows");
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_harmonic_render_bwd(dgc_ctx *ctx, const dgc_harmonic_params *p, const float *f0_dev,
                                           const float *uv_dev, const float *amps_dev, const float *gain_dev,
                                           const float *g_audio_dev, float *scratch_dev, float *g_amps_dev) {
  return harmonic_render_bwd_impl(ctx, p, f0_dev, uv_dev, amps_dev, gain_dev, g_audio_dev, scratch_dev, g_amps_dev, false);
}

DGC_EXPORT int32_t dgc_harmonic_render_bwd_prepared(dgc_ctx *ctx, const dgc_harmonic_params *p, const float *f0_dev,
                                                    const float *uv_dev, const float *amps_dev,
                                                    const float *gain_dev, const float *g_audio_dev,
                                                    float *scratch_dev, float *g_amps_dev) {
  return harmonic_render_bwd_impl(ctx, p, f0_dev, uv_dev, amps_dev, gain_dev, g_audio_dev, scratch_dev, g_amps_dev, true);
}

