// Stateful ops of the reference whose state is a ring of past inputs or a held value, computed FRAME-PARALLEL:
//
//   tensor delay line      Sources/DGen/HigherOps+DelayLine.swift:33-65, emission Sources/DGen/Emit.swift:331-403
//   spectrum delay (fixed and modulated)
//                          Sources/DGen/HigherOps+SpectrumDelay.swift:20-135, emission Sources/DGen/Emit.swift:405-512
//   latch (sample and hold) Sources/DGen/Definitions.swift:104-113, Sources/DGen/Emit+State.swift:225-262
//   compressor             Sources/DGen/HigherOps.swift:566-651
//   phase vocoder          Sources/DGen/HigherOps+PhaseVocoder.swift:15-88, emission Sources/DGen/Emit+PhaseVocoder.swift:6-118
//
// The reference runs each of them in a sequential block, one frame after the other, because they read and write
// a memory cell.  None of the first three is a true recurrence: a delay line's output at frame n is a gather
// from the INPUT at frames n - k and n - k - 1 (the ring only remembers the input), and a latch's output is the
// input at the most recent trigger frame (a prefix maximum over trigger indices).  So every (frame, lane) element
// is one thread; the ring / held-value cells are read for the frames that reach back before the call and
// rewritten at the end of the call so that consecutive calls continue as the reference's persistent cells do.
// The compressor's attack / release smoother IS a recurrence with a data-dependent coefficient (no associative
// form): its gain computer and make-up run sample-parallel in kernels of their own, the smoother runs one warp
// per voice between them.  The phase
// vocoder carries one value per bin from hop to hop (the synthesis phase): its analysis runs parallel over
// (hop, bin), its resynthesis one thread per bin.
#include "common.cuh"

namespace {

// ---- fractional delay gather ----------------------------------------------------------------------------------
// x [T][W]; ring of R past rows (lane-major [W][R] for the delay line, row-major [R][W] for spectra); head = the
// slot the NEXT row is written to.  The row written n frames into the call sits at slot (head + n) mod R, so the
// row k frames before frame n is x[n - k] when n - k >= 0 and ring slot (head + n - k) mod R otherwise.
template <bool ROW_MAJOR>
__device__ __forceinline__ float delayed_sample(const float *__restrict__ x, const float *__restrict__ ring, int w0,
                                                int64_t n, int k, int e, int W, int R) {
  const int64_t m = n - k;
  if (m >= 0) return x[m * W + e];
  if (!ring) return 0.0f;
  int p = (int)(w0 + m);          // m in [-(R-1), -1]
  if (p < 0) p += R;
  return ROW_MAJOR ? ring[(size_t)p * W + e] : ring[(size_t)e * R + p];
}

// delay_mode: -1 fixed integer delay `fixed_k` (no interpolation), 0 one value for the call, 1 per frame [T],
// 2 per frame and lane [T][W], 3 per lane [W]
template <bool ROW_MAJOR>
__global__ void __launch_bounds__(256)
frac_delay_kernel(const float *__restrict__ x, const float *__restrict__ delay, int delay_mode, int fixed_k, int64_t T,
                  int W, int R, float dmax, const float *__restrict__ ring, const float *__restrict__ head,
                  float *__restrict__ y) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * W) return;
  const int64_t n = idx / W;
  const int e = (int)(idx - n * W);
  const int w0 = head ? (int)head[0] : 0;
  if (delay_mode < 0) {
    y[idx] = delayed_sample<ROW_MAJOR>(x, ring, w0, n, fixed_k, e, W, R);
    return;
  }
  const float d = delay_mode == 0 ? delay[0] : delay_mode == 1 ? delay[n] : delay_mode == 2 ? delay[idx] : delay[e];
  const float dc = d > dmax ? dmax : (d < 0.0f ? 0.0f : d);
  const float kf = floorf(dc), frac = dc - kf;
  const int k = (int)kf;
  // the second tap of the longest delay wraps onto the slot written this frame, as the reference's ring does
  int k1 = k + 1;
  if (k1 >= R) k1 -= R;
  const float s0 = delayed_sample<ROW_MAJOR>(x, ring, w0, n, k, e, W, R);
  const float s1 = delayed_sample<ROW_MAJOR>(x, ring, w0, n, k1, e, W, R);
  y[idx] = fmaf(s1, frac, s0 * (1.0f - frac));
}

// The same gather with FOUR lanes per thread (W a multiple of 4, 16-byte aligned rows): the two taps of a frame are
// 128-bit loads and the result one 128-bit streaming store; only frames that reach back into the ring cell, and
// per-lane delay times, fall back to one access per lane.
template <bool ROW_MAJOR>
__device__ __forceinline__ float4 delayed_sample4(const float *__restrict__ x, const float *__restrict__ ring, int w0,
                                                  int64_t n, int k, int e, int W, int R) {
  const int64_t m = n - k;
  if (m >= 0) return __ldg(reinterpret_cast<const float4 *>(x + m * W + e));
  return make_float4(delayed_sample<ROW_MAJOR>(x, ring, w0, n, k, e, W, R),
                     delayed_sample<ROW_MAJOR>(x, ring, w0, n, k, e + 1, W, R),
                     delayed_sample<ROW_MAJOR>(x, ring, w0, n, k, e + 2, W, R),
                     delayed_sample<ROW_MAJOR>(x, ring, w0, n, k, e + 3, W, R));
}

template <bool ROW_MAJOR>
__global__ void __launch_bounds__(256)
frac_delay4_kernel(const float *__restrict__ x, const float *__restrict__ delay, int delay_mode, int fixed_k, int64_t T,
                   int W, int R, float dmax, const float *__restrict__ ring, const float *__restrict__ head,
                   float *__restrict__ y) {
  const int W4 = W >> 2;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, total = T * W4;
  if (idx >= total) return;
  const int64_t n = total <= 0xffffffffLL ? (int64_t)((uint32_t)idx / (uint32_t)W4) : idx / W4;
  const int e = (int)(idx - n * W4) * 4;
  const int w0 = head ? (int)head[0] : 0;
  float4 out;
  if (delay_mode < 0) {
    out = delayed_sample4<ROW_MAJOR>(x, ring, w0, n, fixed_k, e, W, R);
  } else if (delay_mode <= 1) {
    const float d = delay_mode == 0 ? delay[0] : delay[n];
    const float dc = d > dmax ? dmax : (d < 0.0f ? 0.0f : d);
    const float kf = floorf(dc), frac = dc - kf, omf = 1.0f - frac;
    const int k = (int)kf;
    int k1 = k + 1;
    if (k1 >= R) k1 -= R;
    const float4 s0 = delayed_sample4<ROW_MAJOR>(x, ring, w0, n, k, e, W, R);
    const float4 s1 = delayed_sample4<ROW_MAJOR>(x, ring, w0, n, k1, e, W, R);
    out = make_float4(fmaf(s1.x, frac, s0.x * omf), fmaf(s1.y, frac, s0.y * omf), fmaf(s1.z, frac, s0.z * omf),
                      fmaf(s1.w, frac, s0.w * omf));
  } else {
    const float4 d4 = __ldg(reinterpret_cast<const float4 *>(delay_mode == 2 ? delay + n * W + e : delay + e));
    const float dv[4] = {d4.x, d4.y, d4.z, d4.w};
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float dc = dv[j] > dmax ? dmax : (dv[j] < 0.0f ? 0.0f : dv[j]);
      const float kf = floorf(dc), frac = dc - kf;
      const int k = (int)kf;
      int k1 = k + 1;
      if (k1 >= R) k1 -= R;
      const float s0 = delayed_sample<ROW_MAJOR>(x, ring, w0, n, k, e + j, W, R);
      const float s1 = delayed_sample<ROW_MAJOR>(x, ring, w0, n, k1, e + j, W, R);
      o[j] = fmaf(s1, frac, s0 * (1.0f - frac));
    }
    out = make_float4(o[0], o[1], o[2], o[3]);
  }
  __stcs(reinterpret_cast<float4 *>(y + n * W + e), out);
}

template <bool ROW_MAJOR>
static void launch_frac_delay(cudaStream_t st, const float *x, const float *delay, int delay_mode, int fixed_k, int64_t T,
                              int W, int R, float dmax, const float *ring, const float *head, float *y) {
  const bool vec = (W & 3) == 0 && ((((uintptr_t)x) | ((uintptr_t)y) | ((uintptr_t)delay)) & 15) == 0;
  if (vec)
    frac_delay4_kernel<ROW_MAJOR><<<dgc_div_up(T * (W >> 2), 256), 256, 0, st>>>(x, delay, delay_mode, fixed_k, T, W, R, dmax,
                                                                                ring, head, y);
  else
    frac_delay_kernel<ROW_MAJOR><<<dgc_div_up(T * W, 256), 256, 0, st>>>(x, delay, delay_mode, fixed_k, T, W, R, dmax, ring,
                                                                        head, y);
}

// ring slot p holds, after the call, the last row written to it: frames n = off, off + R, ... < T with
// off = (p - head) mod R; untouched when off >= T
template <bool ROW_MAJOR>
__global__ void ring_update_kernel(const float *__restrict__ x, int64_t T, int W, int R, float *__restrict__ ring,
                                   const float *__restrict__ head) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)W * R) return;
  // lanes fastest over threads for the row-major ring, slots fastest for the lane-major one: coalesced writes
  const int e = ROW_MAJOR ? (int)(idx % W) : (int)(idx / R);
  const int p = ROW_MAJOR ? (int)(idx / W) : (int)(idx % R);
  const int w0 = (int)head[0];
  int off = p - w0;
  if (off < 0) off += R;
  if (off >= T) return;
  const int64_t last = off + ((T - 1 - off) / R) * R;
  ring[idx] = x[last * W + e];
}

__global__ void head_advance_kernel(float *head, int64_t T, int R) {
  const int64_t w0 = (int64_t)head[0];
  head[0] = (float)((w0 + T) % R);
}

// ---- latch ------------------------------------------------------------------------------------------------------
constexpr int LATCH_CHUNK = 128;

__device__ __forceinline__ float cond_at(const float *__restrict__ cond, int cond_mode, int64_t n, int e, int W) {
  return cond_mode == 1 ? cond[n] : cond[n * W + e];
}

// last[c][e] = the last frame of chunk c whose trigger is positive, or -1
__global__ void latch_last_kernel(const float *__restrict__ cond, int cond_mode, int64_t T, int W, int NC,
                                  int *__restrict__ last) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
  if (e >= W) return;
  const int64_t n0 = (int64_t)c * LATCH_CHUNK, n1 = min(n0 + (int64_t)LATCH_CHUNK, T);
  int found = -1;
  for (int64_t n = n1 - 1; n >= n0; --n)
    if (cond_at(cond, cond_mode, n, e, W) > 0.0f) {
      found = (int)(n - n0);
      break;
    }
  last[(size_t)c * W + e] = found;
}

// Exclusive "most recent trigger" over chunks in three coalesced steps (threads run along the lanes):
//   segments of LATCH_SEG chunks: (chunk, offset) of the last trigger inside each segment;
//   one thread per lane walks the segment summaries (NC / LATCH_SEG of them) into "most recent before the segment";
//   each (segment, lane) thread then walks its chunks: last[c][e] becomes the offset and src_chunk[c][e] the chunk of
//   the most recent trigger BEFORE chunk c (chunk -1: none yet, the state cell holds the value).
constexpr int LATCH_SEG = 32;

__global__ void latch_seg_kernel(const int *__restrict__ last, int W, int NC, int NS, int *__restrict__ seg_chunk,
                                 int *__restrict__ seg_off) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x, sgm = blockIdx.y;
  if (e >= W) return;
  const int c0 = sgm * LATCH_SEG, c1 = min(c0 + LATCH_SEG, NC);
  int ch = -1, off = 0;
#pragma unroll 8
  for (int c = c0; c < c1; ++c) {
    const int v = last[(size_t)c * W + e];
    if (v >= 0) {
      ch = c;
      off = v;
    }
  }
  seg_chunk[(size_t)sgm * W + e] = ch;
  seg_off[(size_t)sgm * W + e] = off;
}

__global__ void latch_seg_carry_kernel(int *seg_chunk, int *seg_off, int W, int NS) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= W) return;
  int run = -1, run_off = 0;
  for (int sgm = 0; sgm < NS; ++sgm) {
    const int ch = seg_chunk[(size_t)sgm * W + e], off = seg_off[(size_t)sgm * W + e];
    seg_chunk[(size_t)sgm * W + e] = run;
    seg_off[(size_t)sgm * W + e] = run_off;
    if (ch >= 0) {
      run = ch;
      run_off = off;
    }
  }
}

__global__ void latch_carry_kernel(int *last, int *src_chunk, const int *__restrict__ seg_chunk,
                                   const int *__restrict__ seg_off, int W, int NC) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x, sgm = blockIdx.y;
  if (e >= W) return;
  const int c0 = sgm * LATCH_SEG, c1 = min(c0 + LATCH_SEG, NC);
  int run = seg_chunk[(size_t)sgm * W + e], run_off = seg_off[(size_t)sgm * W + e];
#pragma unroll 8
  for (int c = c0; c < c1; ++c) {
    const int here = last[(size_t)c * W + e];
    src_chunk[(size_t)c * W + e] = run;
    last[(size_t)c * W + e] = run_off;
    if (here >= 0) {
      run = c;
      run_off = here;
    }
  }
}

__global__ void latch_out_kernel(const float *__restrict__ value, const float *__restrict__ cond, int cond_mode,
                                 int64_t T, int W, int NC, const int *__restrict__ src_off,
                                 const int *__restrict__ src_chunk, const float *__restrict__ state,
                                 float *__restrict__ y) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
  if (e >= W) return;
  const int sc = src_chunk[(size_t)c * W + e];
  float held = sc >= 0 ? value[((int64_t)sc * LATCH_CHUNK + src_off[(size_t)c * W + e]) * W + e]
                       : (state ? state[e] : 0.0f);
  const int64_t n0 = (int64_t)c * LATCH_CHUNK, n1 = min(n0 + (int64_t)LATCH_CHUNK, T);
  // groups of sixteen frames: all loads of a group are issued before the dependent selects and stores
  constexpr int G = 16;
  for (int64_t n = n0; n < n1; n += G) {
    float v[G], c[G];
#pragma unroll
    for (int j = 0; j < G; ++j) {
      const int64_t m = min(n + j, n1 - 1);
      v[j] = __ldcs(value + m * W + e);
      c[j] = cond_at(cond, cond_mode, m, e, W);
    }
#pragma unroll
    for (int j = 0; j < G; ++j)
      if (n + j < n1) {
        if (c[j] > 0.0f) held = v[j];
        __stcs(y + (n + j) * W + e, held);
      }
  }
}

// The output pass with FOUR lanes per thread (W a multiple of 4): a warp reads 512 contiguous bytes of a frame, the
// block = (W / 4 lane groups) x (chunks) covers whole rows, results leave as 128-bit streaming stores.
__global__ void __launch_bounds__(256)
latch_out4_kernel(const float *__restrict__ value, const float *__restrict__ cond, int cond_mode, int64_t T, int W,
                  int NC, const int *__restrict__ src_off, const int *__restrict__ src_chunk,
                  const float *__restrict__ state, float *__restrict__ y) {
  const int e = (blockIdx.x * blockDim.x + threadIdx.x) * 4, c = blockIdx.y * blockDim.y + threadIdx.y;
  if (e >= W || c >= NC) return;
  float held[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int sc = src_chunk[(size_t)c * W + e + k];
    held[k] = sc >= 0 ? value[((int64_t)sc * LATCH_CHUNK + src_off[(size_t)c * W + e + k]) * W + e + k]
                      : (state ? state[e + k] : 0.0f);
  }
  const int64_t n0 = (int64_t)c * LATCH_CHUNK, n1 = min(n0 + (int64_t)LATCH_CHUNK, T);
  constexpr int G = 8;
  for (int64_t n = n0; n < n1; n += G) {
    float4 v[G], cc[G];
#pragma unroll
    for (int j = 0; j < G; ++j) {
      const int64_t m = min(n + j, n1 - 1);
      v[j] = __ldcs(reinterpret_cast<const float4 *>(value + m * W + e));
      if (cond_mode == 1) {
        const float t = cond[m];
        cc[j] = make_float4(t, t, t, t);
      } else {
        cc[j] = __ldcs(reinterpret_cast<const float4 *>(cond + m * W + e));
      }
    }
#pragma unroll
    for (int j = 0; j < G; ++j)
      if (n + j < n1) {
        if (cc[j].x > 0.0f) held[0] = v[j].x;
        if (cc[j].y > 0.0f) held[1] = v[j].y;
        if (cc[j].z > 0.0f) held[2] = v[j].z;
        if (cc[j].w > 0.0f) held[3] = v[j].w;
        __stcs(reinterpret_cast<float4 *>(y + (n + j) * W + e), make_float4(held[0], held[1], held[2], held[3]));
      }
  }
}

__global__ void latch_state_kernel(const float *__restrict__ y, int64_t T, int W, float *__restrict__ state) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e < W) state[e] = y[(T - 1) * W + e];
}

// ---- compressor -------------------------------------------------------------------------------------------------
struct CompCoef {
  float ratio, threshold, knee, att, rel, knee_start, knee_end, hard_ratio, thr_minus_start;
};

__device__ __forceinline__ float amp2db(float a) { return 20.0f * log10f(fmaxf(fabsf(a), 0.00001f)); }

__device__ __forceinline__ float gain_reduction(const CompCoef &c, float det_db) {
  const float pos = (det_db - c.knee_start) / c.knee;
  const float interp_ratio = 1.0f + pos * (c.ratio - 1.0f);
  const float over = det_db - (c.knee_start + pos * c.thr_minus_start);
  const float soft = over * (1.0f - 1.0f / interp_ratio);
  const float hard = (det_db - c.threshold) * c.hard_ratio;
  return det_db <= c.knee_start ? 0.0f : (det_db >= c.knee_end ? hard : soft);
}

constexpr int COMP_TILE = 256;            // samples per warp iteration: 8 per lane
constexpr int COMP_WARPS = 4;

// pass 1, sample-parallel: gain reduction in dB wanted at every sample (logarithm, knee) -> buf
__global__ void __launch_bounds__(256)
comp_gain_kernel(const float *__restrict__ det, int64_t n, CompCoef c, float *__restrict__ buf) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) buf[i] = gain_reduction(c, amp2db(__ldcs(det + i)));
}

// pass 2, one warp per voice, in place: the attack / release smoother, the one serial dependence of the op.
// Per tile of 256 samples the lanes stage (g, g (1 - att), g (1 - rel)) in shared memory, every lane then walks the
// tile in frame order (per sample: two multiply-adds and a compare side by side, then a select) and keeps the
// smoothed values of its own eight samples for a coalesced store.
__global__ void __launch_bounds__(COMP_WARPS * 32)
comp_smooth_kernel(float *__restrict__ buf, int B, int64_t T, float att, float rel, float *__restrict__ state) {
  __shared__ float4 gs[COMP_WARPS][COMP_TILE];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * COMP_WARPS + warp;
  if (b >= B) return;
  float *gb = buf + (size_t)b * T;
  float s = state ? state[b] : 0.0f;
  const float one_m_att = 1.0f - att, one_m_rel = 1.0f - rel;
  float nxt[COMP_TILE / 32];
#pragma unroll
  for (int j = 0; j < COMP_TILE / 32; ++j) nxt[j] = j * 32 + lane < T ? gb[j * 32 + lane] : 0.0f;
  for (int64_t t0 = 0; t0 < T; t0 += COMP_TILE) {
    const int len = (int)min((int64_t)COMP_TILE, T - t0);
#pragma unroll
    for (int j = 0; j < COMP_TILE / 32; ++j) {
      const float g = nxt[j];
      gs[warp][j * 32 + lane] = make_float4(g, g * one_m_att, g * one_m_rel, 0.0f);
    }
    // the next tile's loads are in flight while this one is walked
    const int64_t t1 = t0 + COMP_TILE;
#pragma unroll
    for (int j = 0; j < COMP_TILE / 32; ++j) nxt[j] = t1 + j * 32 + lane < T ? gb[t1 + j * 32 + lane] : 0.0f;
    __syncwarp();
    float keep[COMP_TILE / 32];
#pragma unroll
    for (int j = 0; j < COMP_TILE / 32; ++j) {
      keep[j] = 0.0f;
      if (j * 32 < len) {                      // uniform over the warp
        const int lim = min(32, len - j * 32);
        if (lim == 32) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float4 g = gs[warp][j * 32 + i];
            const float a_s = fmaf(att, s, g.y), r_s = fmaf(rel, s, g.z);
            s = g.x > s ? a_s : r_s;
            if (i == lane) keep[j] = s;
          }
        } else {
          for (int i = 0; i < lim; ++i) {
            const float4 g = gs[warp][j * 32 + i];
            const float a_s = fmaf(att, s, g.y), r_s = fmaf(rel, s, g.z);
            s = g.x > s ? a_s : r_s;
            if (i == lane) keep[j] = s;
          }
        }
      }
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < COMP_TILE / 32; ++j)
      if (j * 32 + lane < len) gb[t0 + j * 32 + lane] = keep[j];
  }
  if (state && lane == 0) state[b] = s;
}

// pass 3, sample-parallel, in place over the smoothed reduction: y = sign(x) 10^((dB(x) - s) / 20)
__global__ void __launch_bounds__(256)
comp_apply_kernel(const float *__restrict__ x, int64_t n, float *__restrict__ y) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = __ldcs(x + i);
  const float att_db = amp2db(v) - y[i];
  const float amp = powf(10.0f, att_db / 20.0f);
  const float sg = v > 0.0f ? 1.0f : (v < 0.0f ? -1.0f : 0.0f);
  y[i] = sg * amp;
}

// ---- phase vocoder ----------------------------------------------------------------------------------------------
// Emit+PhaseVocoder.swift:46-53
__device__ __forceinline__ float principal_arg(float v) {
  const float tau = 6.28318530717958647692f, half = 3.14159265358979323846f;
  const float w = v - tau * roundf(v / tau);
  const float wh = w > half ? w - tau : w;
  return w < -half ? wh + tau : wh;
}

__device__ __forceinline__ float mixf(float a, float b, float t) { return fmaf(b, t, a * (1.0f - t)); }

// Analysis (Emit+PhaseVocoder.swift:57-71), parallel over (voice, hop, bin): the "previous analysis phase" of hop h
// is the phase of hop h - 1 of the INPUT (the state cell only for the first hop of the call), so nothing here is
// a recurrence.
__global__ void __launch_bounds__(256)
pv_analysis_kernel(const float *__restrict__ re, const float *__restrict__ im, int V, int64_t H, int N, float omega_scale,
                   const float *__restrict__ state, float *__restrict__ mag, float *__restrict__ omega) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)V * H * N) return;
  const int i = (int)(idx % N);
  const int64_t vh = idx / N, h = vh % H;
  const int v = (int)(vh / H);
  const float r = re[idx], q = im[idx];
  const float phase = atan2f(q, r);
  const float prev = h > 0 ? atan2f(im[idx - N], re[idx - N]) : (state ? state[(size_t)v * (2 * N + 1) + i] : 0.0f);
  const float target = (float)i * omega_scale;
  mag[idx] = sqrtf(r * r + q * q);
  omega[idx] = target + principal_arg(phase - prev - target);
}

// Resynthesis (Emit+PhaseVocoder.swift:73-108): thread per (voice, output bin), hops in order: the synthesis phase
// is the one value carried from hop to hop.  ratio_mode 0: one value, 1: [H], 2: [V][H].
__global__ void __launch_bounds__(128)
pv_synthesis_kernel(const float *__restrict__ re, const float *__restrict__ im, const float *__restrict__ mag,
                    const float *__restrict__ omega, const float *__restrict__ ratio, int ratio_mode, int V, int64_t H,
                    int N, float *__restrict__ state, float *__restrict__ out_re, float *__restrict__ out_im) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x, v = blockIdx.y;
  if (k >= N) return;
  float *st = state ? state + (size_t)v * (2 * N + 1) : nullptr;
  float synth = st ? st[N + k] : 0.0f;
  bool started = st ? st[2 * N] != 0.0f : false;
  const float nm1 = (float)(N - 1);
  const size_t base = (size_t)v * H * N;
  for (int64_t h = 0; h < H; ++h) {
    const float rin = ratio_mode == 0 ? ratio[0] : ratio_mode == 1 ? ratio[h] : ratio[(size_t)v * H + h];
    const float r = fmaxf(rin, 1e-4f);
    const float src = (float)k / r;
    const bool in_range = src <= nm1;
    const float srcc = in_range ? src : nm1;
    const float fl = floorf(srcc), frac = srcc - fl;
    const int i0 = (int)fl, i1 = i0 < N - 1 ? i0 + 1 : i0;
    const size_t row = base + (size_t)h * N;
    const float m = mixf(mag[row + i0], mag[row + i1], frac);
    const float om = mixf(omega[row + i0], omega[row + i1], frac) * r;
    if (started) {
      synth = principal_arg(synth + om);
    } else {
      // first hop of the stream: start from the interpolated analysis phase of this hop
      const float p0 = atan2f(im[row + i0], re[row + i0]), p1 = atan2f(im[row + i1], re[row + i1]);
      synth = principal_arg(mixf(p0, p1, frac));
      started = true;
    }
    const float outm = in_range ? m : 0.0f;
    float sn, cs;
    sincosf(synth, &sn, &cs);
    out_re[row + k] = outm * cs;
    out_im[row + k] = outm * sn;
  }
  if (st) {
    const size_t last = base + (size_t)(H - 1) * N + k;
    const float ph = atan2f(im[last], re[last]);
    // the "started" flag is shared by all bins of a voice and other blocks may still have to read it: a launch of
    // its own sets it afterwards
    st[N + k] = synth;
    st[k] = ph;
  }
}

__global__ void pv_mark_started_kernel(float *state, int V, int N) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v < V) state[(size_t)v * (2 * N + 1) + 2 * N] = 1.0f;
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
DGC_EXPORT int32_t dgc_delay_line(dgc_ctx *ctx, const float *x_dev, const float *delay_dev, int32_t delay_mode,
                                  int64_t T, int32_t lanes, int32_t max_delay, float *ring_dev, float *head_dev,
                                  float *y_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, x_dev && delay_dev && y_dev, "null pointer");
  DGC_REQUIRE(ctx, T > 0 && lanes > 0, "size out of range");
  DGC_REQUIRE(ctx, max_delay > 1 && max_delay <= (1 << 24), "max_delay must be in 2..2^24 (the head is a float cell)");
  DGC_REQUIRE(ctx, delay_mode >= 0 && delay_mode <= 3, "delay_mode must be 0 (one value), 1 ([T]), 2 ([T][lanes]) or 3 ([lanes])");
  DGC_REQUIRE(ctx, (ring_dev == nullptr) == (head_dev == nullptr), "ring and head must be given together");
  DGC_REQUIRE(ctx, x_dev != y_dev, "in-place operation is not supported");
  DGC_REQUIRE(ctx, T * lanes / 256 < 0x7fffffffLL, "T * lanes too large");
  launch_frac_delay<false>(ctx->stream, x_dev, delay_dev, delay_mode, 0, T, lanes, max_delay, (float)(max_delay - 1),
                           ring_dev, head_dev, y_dev);
  DGC_LAUNCHED(ctx, "delay_line");
  if (ring_dev) {
    ring_update_kernel<false><<<dgc_div_up((int64_t)lanes * max_delay, 256), 256, 0, ctx->stream>>>(
        x_dev, T, lanes, max_delay, ring_dev, head_dev);
    DGC_LAUNCHED(ctx, "delay_line_ring");
    head_advance_kernel<<<1, 1, 0, ctx->stream>>>(head_dev, T, max_delay);
    DGC_LAUNCHED(ctx, "delay_line_head");
  }
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_spectrum_delay(dgc_ctx *ctx, const float *spec_dev, const float *delay_dev, int64_t H,
                                      int32_t N, int32_t hops, float *ring_dev, float *row_dev, float *out_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, spec_dev && out_dev, "null pointer");
  DGC_REQUIRE(ctx, H > 0 && N > 0, "size out of range");
  DGC_REQUIRE(ctx, hops >= 1 && hops < (1 << 24), "hops must be in 1..2^24-1");
  DGC_REQUIRE(ctx, (ring_dev == nullptr) == (row_dev == nullptr), "ring and row must be given together");
  DGC_REQUIRE(ctx, spec_dev != out_dev, "in-place operation is not supported");
  DGC_REQUIRE(ctx, H * N / 256 < 0x7fffffffLL, "H * N too large");
  const int R = hops + 1;
  // fixed delay: the spectrum of exactly `hops` boundaries ago; modulated: per-hop delay in [0, hops]
  launch_frac_delay<true>(ctx->stream, spec_dev, delay_dev, delay_dev ? 1 : -1, hops, H, N, R, (float)hops, ring_dev,
                          row_dev, out_dev);
  DGC_LAUNCHED(ctx, "spectrum_delay");
  if (ring_dev) {
    ring_update_kernel<true><<<dgc_div_up((int64_t)N * R, 256), 256, 0, ctx->stream>>>(spec_dev, H, N, R, ring_dev,
                                                                                     row_dev);
    DGC_LAUNCHED(ctx, "spectrum_delay_ring");
    head_advance_kernel<<<1, 1, 0, ctx->stream>>>(row_dev, H, R);
    DGC_LAUNCHED(ctx, "spectrum_delay_row");
  }
  return DGC_OK;
}

DGC_EXPORT uint64_t dgc_latch_scratch_floats(int64_t T, int32_t lanes) {
  if (T <= 0 || lanes <= 0) return 0;
  const uint64_t NC = (uint64_t)((T + LATCH_CHUNK - 1) / LATCH_CHUNK), NS = (NC + LATCH_SEG - 1) / LATCH_SEG;
  return (2 * NC + 2 * NS) * (uint64_t)lanes;
}

DGC_EXPORT int32_t dgc_latch(dgc_ctx *ctx, const float *value_dev, const float *cond_dev, int32_t cond_mode, int64_t T,
                             int32_t lanes, float *state_dev, float *scratch_dev, float *y_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, value_dev && cond_dev && y_dev, "null pointer");
  DGC_REQUIRE(ctx, T > 0 && lanes > 0, "size out of range");
  DGC_REQUIRE(ctx, cond_mode == 1 || cond_mode == 2, "cond_mode must be 1 ([T]) or 2 ([T][lanes])");
  const int64_t NC64 = (T + LATCH_CHUNK - 1) / LATCH_CHUNK;
  DGC_REQUIRE(ctx, NC64 <= 65535, "T too large");
  const int NC = (int)NC64;
  float *scr = scratch_dev ? scratch_dev : dgc_ctx_scratch(ctx, dgc_latch_scratch_floats(T, lanes));
  if (!scr) return DGC_ERR_OOM;
  int *last = reinterpret_cast<int *>(scr), *src_chunk = last + (size_t)NC * lanes;
  dim3 grid(dgc_div_up(lanes, 128), NC);
  latch_last_kernel<<<grid, 128, 0, ctx->stream>>>(cond_dev, cond_mode, T, lanes, NC, last);
  DGC_LAUNCHED(ctx, "latch_last");
  const int NS = dgc_div_up(NC, LATCH_SEG);
  int *seg_chunk = src_chunk + (size_t)NC * lanes, *seg_off = seg_chunk + (size_t)NS * lanes;
  dim3 sgrid(dgc_div_up(lanes, 128), NS);
  latch_seg_kernel<<<sgrid, 128, 0, ctx->stream>>>(last, lanes, NC, NS, seg_chunk, seg_off);
  DGC_LAUNCHED(ctx, "latch_segments");
  latch_seg_carry_kernel<<<dgc_div_up(lanes, 128), 128, 0, ctx->stream>>>(seg_chunk, seg_off, lanes, NS);
  DGC_LAUNCHED(ctx, "latch_segment_carry");
  latch_carry_kernel<<<sgrid, 128, 0, ctx->stream>>>(last, src_chunk, seg_chunk, seg_off, lanes, NC);
  DGC_LAUNCHED(ctx, "latch_carry");
  const bool quad = (lanes & 3) == 0 &&
                    ((((uintptr_t)value_dev) | ((uintptr_t)y_dev) | (cond_mode == 2 ? (uintptr_t)cond_dev : 0)) & 15) == 0;
  if (quad) {
    const int bx = lanes / 4 >= 64 ? 64 : lanes / 4, by = 256 / bx >= 1 ? (256 / bx > 8 ? 8 : 256 / bx) : 1;
    latch_out4_kernel<<<dim3(dgc_div_up(lanes / 4, bx), dgc_div_up(NC, by)), dim3(bx, by), 0, ctx->stream>>>(
        value_dev, cond_dev, cond_mode, T, lanes, NC, last, src_chunk, state_dev, y_dev);
  } else {
    latch_out_kernel<<<grid, 128, 0, ctx->stream>>>(value_dev, cond_dev, cond_mode, T, lanes, NC, last, src_chunk,
                                                    state_dev, y_dev);
  }
  DGC_LAUNCHED(ctx, "latch_out");
  if (state_dev) {
    latch_state_kernel<<<dgc_div_up(lanes, 128), 128, 0, ctx->stream>>>(y_dev, T, lanes, state_dev);
    DGC_LAUNCHED(ctx, "latch_state");
  }
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_compressor(dgc_ctx *ctx, const dgc_compressor_params *p, const float *x_dev,
                                  const float *sidechain_dev, float *state_dev, float *y_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, p && x_dev && y_dev, "null pointer");
  DGC_REQUIRE(ctx, p->B > 0 && p->T > 0, "size out of range");
  DGC_REQUIRE(ctx, p->attack > 0.0f && p->release > 0.0f && p->sample_rate > 0.0f, "attack, release and sample_rate must be positive");
  CompCoef c;
  c.ratio = p->ratio;
  c.threshold = p->threshold;
  c.knee = p->knee;
  // exp(log(0.01) / (time * sample_rate)), single precision as the reference graph evaluates it
  const float log001 = logf(0.01f);
  c.att = expf(log001 / (p->attack * p->sample_rate));
  c.rel = expf(log001 / (p->release * p->sample_rate));
  const float half = p->knee / 2.0f;
  c.knee_start = p->threshold - half;
  c.knee_end = p->threshold + half;
  c.hard_ratio = 1.0f - 1.0f / p->ratio;
  c.thr_minus_start = p->threshold - c.knee_start;
  DGC_REQUIRE(ctx, x_dev != y_dev && sidechain_dev != y_dev, "in-place operation is not supported");
  const int64_t n = (int64_t)p->B * p->T;
  DGC_REQUIRE(ctx, n / 256 < 0x7fffffffLL, "B * T too large");
  // y doubles as the work buffer: wanted reduction -> smoothed reduction (in place) -> output (in place)
  comp_gain_kernel<<<dgc_div_up(n, 256), 256, 0, ctx->stream>>>(sidechain_dev ? sidechain_dev : x_dev, n, c, y_dev);
  DGC_LAUNCHED(ctx, "compressor_gain");
  comp_smooth_kernel<<<dgc_div_up(p->B, COMP_WARPS), COMP_WARPS * 32, 0, ctx->stream>>>(y_dev, p->B, p->T, c.att, c.rel,
                                                                                     state_dev);
  DGC_LAUNCHED(ctx, "compressor_smooth");
  comp_apply_kernel<<<dgc_div_up(n, 256), 256, 0, ctx->stream>>>(x_dev, n, y_dev);
  DGC_LAUNCHED(ctx, "compressor");
  return DGC_OK;
}

DGC_EXPORT uint64_t dgc_phase_vocoder_scratch_floats(int32_t V, int64_t H, int32_t N) {
  if (V <= 0 || H <= 0 || N <= 0) return 0;
  return 2ull * (uint64_t)V * (uint64_t)H * (uint64_t)N;
}

DGC_EXPORT int32_t dgc_phase_vocoder(dgc_ctx *ctx, const float *re_dev, const float *im_dev, const float *ratio_dev,
                                     int32_t ratio_mode, int32_t V, int64_t H, int32_t N, int32_t hop, float *state_dev,
                                     float *scratch_dev, float *out_re_dev, float *out_im_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, re_dev && im_dev && ratio_dev && out_re_dev && out_im_dev, "null pointer");
  DGC_REQUIRE(ctx, V > 0 && V <= 65535 && H > 0 && N > 0 && hop > 0, "size out of range");
  DGC_REQUIRE(ctx, ratio_mode >= 0 && ratio_mode <= 2, "ratio_mode must be 0 (one value), 1 ([H]) or 2 ([V][H])");
  DGC_REQUIRE(ctx, re_dev != out_re_dev && im_dev != out_im_dev, "in-place operation is not supported");
  const int64_t total = (int64_t)V * H * N;
  DGC_REQUIRE(ctx, total / 256 < 0x7fffffffLL, "V * H * N too large");
  float *scr = scratch_dev ? scratch_dev : dgc_ctx_scratch(ctx, dgc_phase_vocoder_scratch_floats(V, H, N));
  if (!scr) return DGC_ERR_OOM;
  float *mag = scr, *omega = scr + total;
  const float omega_scale = 2.0f * 3.14159265358979323846f * (float)hop / (float)N;
  pv_analysis_kernel<<<dgc_div_up(total, 256), 256, 0, ctx->stream>>>(re_dev, im_dev, V, H, N, omega_scale, state_dev, mag,
                                                                     omega);
  DGC_LAUNCHED(ctx, "phase_vocoder_analysis");
  pv_synthesis_kernel<<<dim3(dgc_div_up(N, 128), V), 128, 0, ctx->stream>>>(re_dev, im_dev, mag, omega, ratio_dev,
                                                                           ratio_mode, V, H, N, state_dev, out_re_dev,
                                                                           out_im_dev);
  DGC_LAUNCHED(ctx, "phase_vocoder_synthesis");
  if (state_dev) {
    pv_mark_started_kernel<<<dgc_div_up(V, 128), 128, 0, ctx->stream>>>(state_dev, V, N);
    DGC_LAUNCHED(ctx, "phase_vocoder_state");
  }
  return DGC_OK;
}
