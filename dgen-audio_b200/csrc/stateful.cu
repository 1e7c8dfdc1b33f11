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
// form): its gain computer and make-up run sample-parallel, the smoother runs one warp per voice.  The phase
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

// Exclusive "most recent trigger" over chunks, one warp per lane: last[c][e] becomes the chunk index * CHUNK +
// offset of the most recent trigger BEFORE chunk c, as a 64-bit frame index split over two int planes
// (plane 0: chunk of the trigger or -1, plane 1: offset within it).
__global__ void latch_carry_kernel(int *last, int *src_chunk, int W, int NC) {
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (e >= W) return;
  const int seg = (NC + 31) / 32, c0 = lane * seg, c1 = min(c0 + seg, NC);
  // most recent trigger chunk within this thread's segment
  int mine = -1;
  for (int c = c0; c < c1; ++c)
    if (last[(size_t)c * W + e] >= 0) mine = c;
  // exclusive prefix maximum across the warp (chunk indices grow with the segment)
  int incl = mine;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    int o = __shfl_up_sync(0xffffffffu, incl, s);
    if (lane >= s) incl = max(incl, o);
  }
  int run = __shfl_up_sync(0xffffffffu, incl, 1);
  if (lane == 0) run = -1;
  int run_off = run >= 0 ? last[(size_t)run * W + e] : 0;   // read before any thread overwrites: see the sync below
  __syncwarp();
  // every thread has read the offsets it needs from other segments; within its own segment it reads ahead of
  // what it writes
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
#pragma unroll 4
  for (int64_t n = n0; n < n1; ++n) {
    const float v = value[n * W + e];
    if (cond_at(cond, cond_mode, n, e, W) > 0.0f) held = v;
    y[n * W + e] = held;
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

// one warp per voice.  Per tile: the lanes evaluate the gain computer of their eight samples (logarithm, knee),
// every lane then walks the 256 smoothed values in frame order from shared memory (the one serial dependence:
// compare, two multiply-adds, select) and keeps those of its own samples, and the lanes apply the gain.
__global__ void __launch_bounds__(COMP_WARPS * 32)
compressor_kernel(const float *__restrict__ x, const float *__restrict__ side, int B, int64_t T, CompCoef c,
                  float *__restrict__ state, float *__restrict__ y) {
  __shared__ float4 gs[COMP_WARPS][COMP_TILE];   // (g, g (1 - att), g (1 - rel), unused)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * COMP_WARPS + warp;
  if (b >= B) return;
  const float *xb = x + (size_t)b * T, *db = side ? side + (size_t)b * T : xb;
  float *yb = y + (size_t)b * T;
  float s = state ? state[b] : 0.0f;
  const float one_m_att = 1.0f - c.att, one_m_rel = 1.0f - c.rel;
  for (int64_t t0 = 0; t0 < T; t0 += COMP_TILE) {
    const int len = (int)min((int64_t)COMP_TILE, T - t0);
    float xv[COMP_TILE / 32];
#pragma unroll
    for (int j = 0; j < COMP_TILE / 32; ++j) {
      const int i = j * 32 + lane;
      xv[j] = i < len ? xb[t0 + i] : 0.0f;
      const float dv = i < len ? db[t0 + i] : 0.0f;
      const float g = gain_reduction(c, amp2db(dv));
      gs[warp][i] = make_float4(g, g * one_m_att, g * one_m_rel, 0.0f);
    }
    __syncwarp();
    float keep[COMP_TILE / 32];
#pragma unroll
    for (int j = 0; j < COMP_TILE / 32; ++j) {
      if (j * 32 < len) {                      // uniform over the warp
        const int lim = min(32, len - j * 32);
#pragma unroll 8
        for (int i = 0; i < lim; ++i) {
          const float4 g = gs[warp][j * 32 + i];
          const float a_s = fmaf(c.att, s, g.y), r_s = fmaf(c.rel, s, g.z);
          s = g.x > s ? a_s : r_s;
          if (i == lane) keep[j] = s;
        }
      }
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < COMP_TILE / 32; ++j) {
      const int i = j * 32 + lane;
      if (i < len) {
        const float v = xv[j];
        const float att_db = amp2db(v) - keep[j];
        const float amp = powf(10.0f, att_db / 20.0f);
        const float sg = v > 0.0f ? 1.0f : (v < 0.0f ? -1.0f : 0.0f);
        yb[t0 + i] = sg * amp;
      }
    }
  }
  if (state && lane == 0) state[b] = s;
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
  frac_delay_kernel<false><<<dgc_div_up(T * lanes, 256), 256, 0, ctx->stream>>>(
      x_dev, delay_dev, delay_mode, 0, T, lanes, max_delay, (float)(max_delay - 1), ring_dev, head_dev, y_dev);
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
  frac_delay_kernel<true><<<dgc_div_up(H * N, 256), 256, 0, ctx->stream>>>(
      spec_dev, delay_dev, delay_dev ? 1 : -1, hops, H, N, R, (float)hops, ring_dev, row_dev, out_dev);
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
  return 2ull * (uint64_t)((T + LATCH_CHUNK - 1) / LATCH_CHUNK) * (uint64_t)lanes;
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
  latch_carry_kernel<<<dgc_div_up(lanes, 4), 128, 0, ctx->stream>>>(last, src_chunk, lanes, NC);
  DGC_LAUNCHED(ctx, "latch_carry");
  latch_out_kernel<<<grid, 128, 0, ctx->stream>>>(value_dev, cond_dev, cond_mode, T, lanes, NC, last, src_chunk,
                                                  state_dev, y_dev);
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
  compressor_kernel<<<dgc_div_up(p->B, COMP_WARPS), COMP_WARPS * 32, 0, ctx->stream>>>(x_dev, sidechain_dev, p->B, p->T, c,
                                                                                    state_dev, y_dev);
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
