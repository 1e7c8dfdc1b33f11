// Multi-scale spectral loss (forward and backward) fused with windowing and magnitude.
//
// Reference semantics (Sources/DGen/Emit+SpectralLoss.swift:719-938): at every hop frame f the
// window s[n] = x[f-(N-1)+n] * hann[n] (zero outside [0,T)) of both signals is transformed, the
// magnitudes of bins 0..N/2 are compared (L1 on |X| and L1 on log(|X|+eps)), summed over bins per
// (hop frame, voice), averaged over voices.  The reference runs one thread per (hop frame, voice)
// and one kernel per term; here one block transforms several windows cooperatively in shared
// memory, prediction and target ride the real and imaginary lane of ONE complex FFT, and the
// linear and log terms come from the same spectrum.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "common.cuh"
#include "fft.cuh"
#include "fft16.cuh"
#include "tma.cuh"

namespace {

using namespace dgfft;

constexpr int LOSS_THREADS = 256;
constexpr float LOG_EPS = 1e-8f;  // DGenSpectralConfig.logMagnitudeEpsilon, Sources/DGen/GradientConfig.swift:38

// Sum `v` over the G = N/8 threads that carry one transform (G is a power of two).  `red` is a
// shared array of one float per warp of the block.  Result valid in the group's first thread.
template <int G>
__device__ __forceinline__ float group_sum(float v, float *red, int tid) {
  constexpr int W = G < 32 ? G : 32;
#pragma unroll
  for (int off = W / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if (G > 32) {
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    if ((tid & (G - 1)) == 0) {
      float s = 0.0f;
#pragma unroll
      for (int w = 0; w < G / 32; ++w) s += red[(tid >> 5) + w];
      v = s;
    }
  }
  return v;
}

// Unpack the spectra of two real signals from the transform of z = x1 + i x2.
__device__ __forceinline__ void unpack(float2 zk, float2 znk, float2 &x1, float2 &x2) {
  x1 = make_float2(0.5f * (zk.x + znk.x), 0.5f * (zk.y - znk.y));
  x2 = make_float2(0.5f * (zk.y + znk.y), 0.5f * (znk.x - zk.x));
}

// One block of one scale: LOSS_THREADS / (N/8) windows of one voice, prediction and target in the real
// and imaginary lane of one transform; sm holds 2 * NF * padded(N) float2 (the same 34.8 KB for every N).
template <int N, bool SUM2>
__device__ __forceinline__ void mss_fwd_body(float2 *sm, float *red, int bx, int b, const float *__restrict__ pred,
                                             const float *__restrict__ pred_b,
                                             const float *__restrict__ target, int B, int T, int hop, int H,
                                             const float *__restrict__ window, const float2 *__restrict__ tw,
                                             float *__restrict__ part_lin, float *__restrict__ part_log) {
  constexpr int G = N / 8;                    // threads per transform
  constexpr int NF = LOSS_THREADS / G;        // transforms per block
  constexpr int PN = padded(N);
  float2 *bufa = sm, *bufb = sm + NF * PN;
  const int tid = threadIdx.x, f = tid / G, lt = tid % G;
  const int h = bx * NF + f;
  const bool valid = h < H;
  const int t_base = h * hop - (N - 1);
  const float *x1 = pred + (size_t)b * T, *x2 = target + (size_t)b * T;
  const float *x1b = SUM2 ? pred_b + (size_t)b * T : nullptr;   // prediction given as a sum of two signals
  float2 *a = bufa + f * PN, *bb = bufb + f * PN;
  // the windowed samples a thread loads (stride G) are exactly its inputs of the first radix-8 stage: they stay
  // in registers
  float2 vin[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    int i = lt + q * G, t = t_base + i;
    float2 v = make_float2(0.0f, 0.0f);
    if (valid && t >= 0 && t < T) {
      float w = __ldg(&window[i]);
      const float xp = SUM2 ? __fadd_rn(x1[t], x1b[t]) : x1[t];
      v = make_float2(xp * w, x2[t] * w);
    }
    vin[q] = v;
  }
  float2 *z = fft_block_regs<N, false>(vin, a, bb, lt, tw);
  float lin = 0.0f, lg = 0.0f;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    int k = lt + q * G;  // 0 .. N/2-1
    float2 X1, X2;
    unpack(z[pad(k)], z[pad((N - k) & (N - 1))], X1, X2);
    float m1 = sqrtf(X1.x * X1.x + X1.y * X1.y), m2 = sqrtf(X2.x * X2.x + X2.y * X2.y);
    lin += fabsf(m1 - m2);
    lg += fabsf(__logf(m1 + LOG_EPS) - __logf(m2 + LOG_EPS));
  }
  if (lt == 0) {  // Nyquist bin
    float2 zn = z[pad(N / 2)];
    float m1 = fabsf(zn.x), m2 = fabsf(zn.y);
    lin += fabsf(m1 - m2);
    lg += fabsf(__logf(m1 + LOG_EPS) - __logf(m2 + LOG_EPS));
  }
  lin = group_sum<G>(lin, red, tid);
  lg = group_sum<G>(lg, red, tid);
  if (valid && lt == 0) {
    part_lin[(size_t)h * B + b] = lin;
    part_log[(size_t)h * B + b] = lg;
  }
}

// All scales of the multi-scale loss in ONE launch: blockIdx.x runs through the blocks of scale 0, then
// scale 1, ... (the host orders the scales by decreasing window so the long blocks start first and the
// short ones fill the tail); no launch gap and no partial last wave per scale.
struct FwdDesc {
  int nscales;
  int N[DGC_MSS_MAX_SCALES], hop[DGC_MSS_MAX_SCALES], H[DGC_MSS_MAX_SCALES];
  int first_block[DGC_MSS_MAX_SCALES + 1];
  const float *window[DGC_MSS_MAX_SCALES];
  const float2 *tw[DGC_MSS_MAX_SCALES];
  float *lin[DGC_MSS_MAX_SCALES], *lg[DGC_MSS_MAX_SCALES];
};

constexpr int FWD_SMEM_BYTES = 2 * (LOSS_THREADS / (2048 / 8)) * padded(2048) * (int)sizeof(float2);

template <bool SUM2>
__global__ void __launch_bounds__(LOSS_THREADS, 6)
mss_fwd_kernel(const float *__restrict__ pred, const float *__restrict__ pred_b, const float *__restrict__ target,
               int B, int T, const FwdDesc d) {
  extern __shared__ float2 fwd_sm[];
  __shared__ float red[LOSS_THREADS / 32];
  int s = 0;
  while (s + 1 < d.nscales && (int)blockIdx.x >= d.first_block[s + 1]) ++s;
  const int bx = blockIdx.x - d.first_block[s], b = blockIdx.y;
  switch (d.N[s]) {
#define CASE(NN) \
  case NN: mss_fwd_body<NN, SUM2>(fwd_sm, red, bx, b, pred, pred_b, target, B, T, d.hop[s], d.H[s], d.window[s], d.tw[s], d.lin[s], d.lg[s]); break;
    CASE(16) CASE(32) CASE(64) CASE(128) CASE(256) CASE(512) CASE(1024) CASE(2048)
#undef CASE
    default: break;
  }
}

// ---------------------------------------------------------------------------------------------
// Forward, register-blocked: sixteen points per thread (fft16.cuh), N/16 threads per window, 128-thread
// blocks.  A thread loads its sixteen windowed samples of both signals straight into the registers of the
// first radix-16 (or radix-8) stage, the transform exchanges through shared memory twice (once for N <= 128),
// and the last stage leaves bin k and bin N - k in the SAME thread, so the spectra of the two real signals are
// unpacked, compared and summed without another pass over shared memory.  The factor 1/2 of the unpacking is
// carried as 2 |X|: the linear term is halved once at the end, and log(2|X| + 2 eps) - log(2|Y| + 2 eps) is the
// reference's log(|X| + eps) - log(|Y| + eps); square roots and logarithms are the approximate hardware ones.
// ---------------------------------------------------------------------------------------------
constexpr int LOSS16_THREADS = 128;
constexpr float LN2_F = 0.69314718055994531f;

__device__ __forceinline__ float fast_sqrt(float v) {
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

// one {k, N - k} pair of bins of z = FFT(x1 + i x2): adds 2 | |X1| - |X2| | and the log2 term
__device__ __forceinline__ void pair_terms(float2 zk, float2 zn, float &lin, float &lg) {
  const float ax = zk.x + zn.x, ay = zk.y - zn.y;     // 2 X1[k]
  const float bx = zk.y + zn.y, by = zn.x - zk.x;     // 2 X2[k]
  const float m1 = fast_sqrt(fmaf(ax, ax, ay * ay)), m2 = fast_sqrt(fmaf(bx, bx, by * by));
  lin += fabsf(m1 - m2);
  lg += fabsf(__log2f(m1 + 2.0f * LOG_EPS) - __log2f(m2 + 2.0f * LOG_EPS));
}
// (a bin that is its own partner, k = 0 or k = N/2, is the pair (z, z): 2 X1 = 2 Re z, 2 X2 = 2 Im z)

// boxes of the staged sample run (TMA variant): SPAN_BOX floats wide, at most SPAN_BOXES of them per signal; the
// two signals' runs share the second transform buffer, which the transform does not touch before its middle stage
constexpr int SPAN_BOX = 128, SPAN_BOXES = 17;
static_assert(2 * SPAN_BOX * SPAN_BOXES * sizeof(float) <= padded(2048) * sizeof(float2), "the staged runs must fit the buffer");

template <int N, bool SUM2, bool TMA>
__device__ __forceinline__ void mss_fwd16_body(float2 *sm, float *red, int bx, int b, const float *__restrict__ pred,
                                               const float *__restrict__ pred_b,
                                               const float *__restrict__ target, int B, int T, int hop, int H,
                                               const float *__restrict__ window, const float2 *__restrict__ tw,
                                               float *__restrict__ part_lin, float *__restrict__ part_log,
                                               const CUtensorMap *map_pred, const CUtensorMap *map_target,
                                               uint64_t *bar, int32_t *status) {
  using Gm = dgfft16::Geo<N>;
  constexpr int TT = Gm::T;                     // threads per window
  constexpr int NF = LOSS16_THREADS / TT;       // windows per block
  // conflict-free layouts for the in-place transform; the copy-engine variant keeps the classic two-buffer form
  using Lay = typename std::conditional<TMA, dgfft16::LayoutClassic, dgfft16::LayoutFree>::type;
  constexpr int PN = Lay::template size<N>(), RL = Gm::RL;
  const int tid = threadIdx.x, f = tid / TT, lt = tid % TT;
  const int h = bx * NF + f;
  const bool valid = h < H;
  const int t_base = h * hop - (N - 1);
  const float *x1 = pred + (size_t)b * T, *x2 = target + (size_t)b * T;
  const float *x1b = SUM2 ? pred_b + (size_t)b * T : nullptr;   // prediction given as a sum of two signals
  // one buffer per transform (in-place middle stage): 17 KB per block instead of 33, room for 8 resident blocks;
  // the variant that stages the sample runs with the copy engine keeps the second buffer for them
  float2 *bufa = sm + f * PN, *bufb = TMA ? sm + (NF + f) * PN : bufa;
  float2 x[16];
  if (TMA) {
    // The run of samples the block's NF windows cover, fetched once by the copy engine: boxes of SPAN_BOX floats
    // from column x0 = the first window's start rounded down to a multiple of 4 (16 bytes).  Columns before the
    // start of the signal arrive as zeros, so no thread tests a bound; a window ends at frame h hop <= T - 1.
    float *span1 = reinterpret_cast<float *>(sm + NF * PN), *span2 = span1 + SPAN_BOX * SPAN_BOXES;
    const int tb0 = (bx * NF) * hop - (N - 1);
    const int x0 = tb0 & ~3;
    const int span = (NF - 1) * hop + N + (tb0 - x0);
    const int nbox = (span + SPAN_BOX - 1) / SPAN_BOX;          // <= SPAN_BOXES whenever hop <= N
    if (tid < 32) {   // the first warp: one lane announces the bytes, then the lanes issue one box each
      if (tid == 0) dgtma::mbar_expect_tx(bar, 2u * nbox * SPAN_BOX * sizeof(float));
      __syncwarp();
      for (int k = tid; k < 2 * nbox; k += 32) {
        const int kb = k >> 1;
        dgtma::load_2d((k & 1 ? span2 : span1) + kb * SPAN_BOX, (k & 1) ? map_target : map_pred, x0 + kb * SPAN_BOX, b, bar);
      }
    }
    // one decision for the whole block (a wait that gave up in one thread must not leave the others at a barrier)
    const bool arrived = __syncthreads_and(dgtma::mbar_wait(bar, 0));
    if (!arrived) {   // the copies never completed: report, and leave without touching the buffers
      if (tid == 0) atomicExch(status, 102);
      return;
    }
    const int off = (tb0 - x0) + f * hop + lt;
    const float *wp = window + lt;
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      const float w = valid ? __ldg(wp + m * TT) : 0.0f;
      x[m] = make_float2(span1[off + m * TT] * w, span2[off + m * TT] * w);
    }
    __syncthreads();   // every warp has read its samples before any transform writes into that buffer
  } else
  // a window ends at frame h * hop <= T - 1, so only its start can fall outside the signal
  if (valid && t_base >= 0) {
    const float *p1 = x1 + t_base + lt, *p2 = x2 + t_base + lt, *wp = window + lt;
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      const float w = __ldg(wp + m * TT);
      const float xp = SUM2 ? __fadd_rn(p1[m * TT], x1b[t_base + lt + m * TT]) : p1[m * TT];
      x[m] = make_float2(xp * w, p2[m * TT] * w);
    }
  } else {
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      const int i = lt + m * TT, t = t_base + i;
      float2 v = make_float2(0.0f, 0.0f);
      if (valid && t >= 0) {
        const float w = __ldg(&window[i]);
        const float xp = SUM2 ? __fadd_rn(x1[t], x1b[t]) : x1[t];
        v = make_float2(xp * w, x2[t] * w);
      }
      x[m] = v;
    }
  }
  float2 z[Gm::PAIRS][2][RL];
  dgfft16::fft16<N, false, Lay>(x, z, bufa, bufb, lt, tw);
  float lin = 0.0f, lg = 0.0f;
  // Bin pairs {k, N - k}.  A pair of butterflies (a, N/RL - a) gives RL of them: bin t of the first with bin
  // RL - 1 - t of the second.  The one thread that holds butterflies 0 and N/(2 RL) instead pairs bins INSIDE each
  // (0 and N/2 with themselves, t with RL - t; t with RL - 1 - t): RL + 1 terms.  Both cases run the same
  // instructions on operands picked by a select, so the warp does not execute the terms twice.
  const bool sp = lt == 0;      // only pair 0 of local thread 0 is the special one
#pragma unroll
  for (int p = 0; p < Gm::PAIRS; ++p) {
    if (p > 0) {
#pragma unroll
      for (int t = 0; t < RL; ++t) pair_terms(z[p][0][t], z[p][1][RL - 1 - t], lin, lg);
    } else {
#pragma unroll
      for (int t = 0; t < RL; ++t) {
        const float2 ks = t <= RL / 2 ? z[0][0][t] : z[0][1][t - RL / 2 - 1];
        const float2 ns = t == 0 ? z[0][0][0] : t < RL / 2 ? z[0][0][RL - t] : t == RL / 2 ? z[0][0][RL / 2]
                                                                                            : z[0][1][RL - 1 - (t - RL / 2 - 1)];
        const float2 kg = z[0][0][t], ng = z[0][1][RL - 1 - t];
        const float2 zk = make_float2(sp ? ks.x : kg.x, sp ? ks.y : kg.y);
        const float2 zn = make_float2(sp ? ns.x : ng.x, sp ? ns.y : ng.y);
        pair_terms(zk, zn, lin, lg);
      }
      if (sp) pair_terms(z[0][1][RL / 2 - 1], z[0][1][RL / 2], lin, lg);
    }
  }
  lin = group_sum<TT>(lin, red, tid);
  lg = group_sum<TT>(lg, red, tid);
  if (valid && lt == 0) {
    part_lin[(size_t)h * B + b] = 0.5f * lin;
    part_log[(size_t)h * B + b] = LN2_F * lg;
  }
}

// 128 threads of transforms per block: the largest of NF * size<N>() over the sizes is 32 x 76 elements (N = 64);
// the copy-engine variant uses two classic buffers of padded(2048)
constexpr int FWD16_SMEM_BYTES = 32 * 76 * (int)sizeof(float2);
static_assert(FWD16_SMEM_BYTES >= padded(2048) * (int)sizeof(float2) && FWD16_SMEM_BYTES >= 4 * 568 * (int)sizeof(float2) &&
              FWD16_SMEM_BYTES >= 8 * 280 * (int)sizeof(float2), "one buffer per transform must fit");

template <bool SUM2, bool TMA>
__global__ void __launch_bounds__(LOSS16_THREADS, TMA ? 6 : 8)
mss_fwd16_kernel(const float *__restrict__ pred, const float *__restrict__ pred_b, const float *__restrict__ target,
                 int B, int T, const FwdDesc d, const __grid_constant__ CUtensorMap map_pred,
                 const __grid_constant__ CUtensorMap map_target, int32_t *status) {
  extern __shared__ __align__(128) float2 fwd_sm[];
  __shared__ float red[LOSS16_THREADS / 32];
  __shared__ __align__(8) uint64_t span_bar;
  if (TMA) {
    if (threadIdx.x == 0) dgtma::mbar_init(&span_bar, 1);
    __syncthreads();
  }
  // one-dimensional grid, scale-major: first_block[s] counts the blocks of ALL voices of the scales before s, so
  // the blocks resident on an SM at any time run the same window size (the same instructions) except at the
  // boundary between two scales
  int s = 0;
  while (s + 1 < d.nscales && (int)blockIdx.x >= d.first_block[s + 1]) ++s;
  const int r = blockIdx.x - d.first_block[s];
  const int per_voice = (d.first_block[s + 1] - d.first_block[s]) / B;
  const int b = r / per_voice, bx = r - b * per_voice;
  switch (d.N[s]) {
#define CASE(NN) \
  case NN: mss_fwd16_body<NN, SUM2, TMA>(fwd_sm, red, bx, b, pred, pred_b, target, B, T, d.hop[s], d.H[s], d.window[s], d.tw[s], d.lin[s], d.lg[s], &map_pred, &map_target, &span_bar, status); break;
    CASE(64) CASE(128) CASE(256) CASE(512) CASE(1024) CASE(2048)
#undef CASE
    default: break;
  }
}

// total = sum_s (w_lin * sum(lin_s) + w_log * sum(log_s)) / B / nscales / T
struct ReduceDesc {
  int nscales;
  long long off[DGC_MSS_MAX_SCALES];  // offset of the lin block of scale s; log block follows
  long long cnt[DGC_MSS_MAX_SCALES];  // H_s * B
};

constexpr int RED_BLOCKS = 256, RED_THREADS = 256;

// Stage 1: every block sums a strided share of all partials (weighted) in double, in a fixed
// order; the last block to finish (ticket counter) adds the RED_BLOCKS block sums by the same fixed tree.
// The result therefore does not depend on scheduling.
__global__ void __launch_bounds__(RED_THREADS)
mss_reduce_kernel(const float *__restrict__ part, ReduceDesc d, double scale_lin, double scale_log,
                  double *__restrict__ block_sums, unsigned int *__restrict__ ticket, double *__restrict__ out) {
  __shared__ double sh[RED_THREADS];
  __shared__ bool last;
  double acc = 0.0;
  const long long stride = (long long)RED_BLOCKS * RED_THREADS;
  for (int s = 0; s < d.nscales; ++s) {
    const float *lin = part + d.off[s], *lg = lin + d.cnt[s];
    double a = 0.0, c = 0.0;
    for (long long i = (long long)blockIdx.x * RED_THREADS + threadIdx.x; i < d.cnt[s]; i += stride) {
      a += (double)lin[i];
      c += (double)lg[i];
    }
    acc += a * scale_lin + c * scale_log;
  }
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (int off = RED_THREADS / 2; off > 0; off >>= 1) {
    if (threadIdx.x < off) sh[threadIdx.x] += sh[threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    block_sums[blockIdx.x] = sh[0];
    __threadfence();
    last = atomicAdd(ticket, 1u) == RED_BLOCKS - 1;
  }
  __syncthreads();
  if (last) {   // the same fixed tree over the block sums, whichever block comes last
    static_assert(RED_BLOCKS == RED_THREADS, "one block sum per thread of the last block");
    __threadfence();
    sh[threadIdx.x] = reinterpret_cast<volatile double *>(block_sums)[threadIdx.x];
    __syncthreads();
    for (int off = RED_THREADS / 2; off > 0; off >>= 1) {
      if (threadIdx.x < off) sh[threadIdx.x] += sh[threadIdx.x + off];
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      out[0] = sh[0];
      *ticket = 0u;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Backward.  Reference: three kernels per term with device scratch for the spectra, the spectral
// gradient and the time gradient (Sources/DGen/Emit+SpectralLoss.swift:940-1325):
//   gradMag1 = sign(d) (* 1/(m1+eps) for the log term) * upstream / B ; gradX1 = gradMag1 * X1 / max(m1, 1e-8)
//   for bins 0..N/2, zero above; time gradient = Re(sum_k gradX1[k] e^{+2 pi i k n / N}) * hann[n];
//   d loss / d x[p] = sum of the time gradients of the hop windows that cover p.
// Here nothing is stored: a block owns a run of output frames, recomputes the spectra of every window
// that covers them (prediction and target in one transform), builds the Hermitian-symmetrised
// spectral gradient of two windows in the real / imaginary lane of one inverse transform, and sums
// the covering windows into a shared-memory tile in a fixed order (rounds ascending, windows
// ascending), so the result is bit-reproducible and needs no atomics.
// ---------------------------------------------------------------------------------------------
template <int N>
struct BwdGeom {
  static constexpr int G = N / 8;
  static constexpr int NF = LOSS_THREADS / G;                      // window pairs per round
  static constexpr int WR = 2 * NF;                                // windows per round
  static constexpr int ROUNDS = WR >= 16 ? 1 : 16 / WR;            // at least 16 windows per block
  static constexpr int WB = WR * ROUNDS;                           // windows per block
};

__device__ __forceinline__ float sgn(float v) { return v > 0.f ? 1.f : (v < 0.f ? -1.f : 0.f); }

// at least three resident blocks per SM for the large windows (caps the registers at 80; the kernel is latency
// bound at the two blocks it would otherwise get), four for the small ones (which need fewer registers anyway)
template <int N>
__global__ void __launch_bounds__(LOSS_THREADS, (N >= 256 ? 3 : 4))
mss_bwd_kernel(const float *__restrict__ pred, const float *__restrict__ target, int B, int T, int hop, int H,
               int S /* windows whose first-covered frames this block owns */, const float *__restrict__ window,
               const float2 *__restrict__ tw, float c_lin, float c_log, int accumulate, float *__restrict__ grad) {
  using Gm = BwdGeom<N>;
  constexpr int G = Gm::G, NF = Gm::NF, WR = Gm::WR;
  extern __shared__ float2 sm2[];
  constexpr int PN = padded(N);
  float2 *bufa = sm2, *bufb = sm2 + NF * PN, *bufg = sm2 + 2 * NF * PN;
  float *tile = reinterpret_cast<float *>(sm2 + 3 * NF * PN);
  const int tid = threadIdx.x, f = tid / G, lt = tid % G;
  const int b = blockIdx.y;
  const int hA = blockIdx.x * S;
  const int p0 = (hA - 1) * hop + 1;          // first owned frame (may be negative for the first block)
  const int owned = S * hop;
  const float *x1 = pred + (size_t)b * T, *x2 = target + (size_t)b * T;
  float2 *a = bufa + f * PN, *bb = bufb + f * PN, *gi = bufg + f * PN;
  for (int o = tid; o < owned; o += LOSS_THREADS) tile[o] = 0.0f;
  const int E = (N - 1) / hop;
  const int nwin = min(S + E, H - hA);        // windows this block must visit
  for (int r0 = 0; r0 < nwin; r0 += WR) {
    const int hr0 = hA + r0;
#pragma unroll
    for (int q = 0; q < 8; ++q) gi[pad(lt + q * G)] = make_float2(0.f, 0.f);
    for (int w = 0; w < 2; ++w) {
      const int h = hr0 + 2 * f + w;
      const bool valid = h < H && (h - hA) < nwin;
      const int t_base = h * hop - (N - 1);
      float2 vin[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        int i = lt + q * G, t = t_base + i;
        float2 v = make_float2(0.f, 0.f);
        if (valid && t >= 0 && t < T) {
          float wv = __ldg(&window[i]);
          v = make_float2(x1[t] * wv, x2[t] * wv);
        }
        vin[q] = v;
      }
      float2 *z = fft_block_regs<N, false>(vin, a, bb, lt, tw);
      if (valid) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          int k = lt + q * G;
          float2 X1, X2;
          unpack(z[pad(k)], z[pad((N - k) & (N - 1))], X1, X2);
          float m1 = sqrtf(X1.x * X1.x + X1.y * X1.y), m2 = sqrtf(X2.x * X2.x + X2.y * X2.y);
          float ld = __logf(m1 + LOG_EPS) - __logf(m2 + LOG_EPS);
          float gm = c_lin * sgn(m1 - m2) + c_log * sgn(ld) / (m1 + LOG_EPS);
          float sc = gm / fmaxf(m1, 1e-8f);
          float2 gk = make_float2(sc * X1.x, sc * X1.y);
          if (k == 0) {
            // a real bin: only Re contributes to the real part of the synthesis
            if (w == 0) gi[0].x += gk.x; else gi[0].y += gk.x;  // pad(0) == 0
          } else {
            float2 hk = make_float2(0.5f * gk.x, 0.5f * gk.y);
            if (w == 0) {
              gi[pad(k)].x += hk.x; gi[pad(k)].y += hk.y;
              gi[pad(N - k)].x += hk.x; gi[pad(N - k)].y -= hk.y;
            } else {  // times i: (x, y) -> (-y, x)
              gi[pad(k)].x -= hk.y; gi[pad(k)].y += hk.x;
              gi[pad(N - k)].x += hk.y; gi[pad(N - k)].y += hk.x;
            }
          }
        }
        if (lt == 0) {
          float2 zn = z[pad(N / 2)];
          float m1 = fabsf(zn.x), m2 = fabsf(zn.y);
          float ld = __logf(m1 + LOG_EPS) - __logf(m2 + LOG_EPS);
          float gm = c_lin * sgn(m1 - m2) + c_log * sgn(ld) / (m1 + LOG_EPS);
          float gre = gm / fmaxf(m1, 1e-8f) * zn.x;
          if (w == 0) gi[pad(N / 2)].x += gre; else gi[pad(N / 2)].y += gre;
        }
      }
      __syncthreads();
    }
    float2 *zt = fft_block<N, true>(gi, a, lt, tw);
    const bool in_g = (zt == gi);  // uniform: depends on the stage count of N only
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      int i = lt + q * G;
      float wv = __ldg(&window[i]);
      zt[pad(i)] = make_float2(zt[pad(i)].x * wv, zt[pad(i)].y * wv);
    }
    __syncthreads();
    const float2 *res = in_g ? bufg : bufa;
    for (int o = tid; o < owned; o += LOSS_THREADS) {
      int p = p0 + o;
      if (p < 0 || p >= T) continue;
      int hlo = max(hr0, (p + hop - 1) / hop);
      int hhi = min(min(hr0 + WR - 1, (p + N - 1) / hop), min(H - 1, hA + nwin - 1));
      float acc = tile[o];
      for (int h = hlo; h <= hhi; ++h) {
        int slot = h - hr0;
        float2 v = res[(slot >> 1) * PN + pad(p - (h * hop - (N - 1)))];
        acc += (slot & 1) ? v.y : v.x;
      }
      tile[o] = acc;
    }
    __syncthreads();
  }
  float *g = grad + (size_t)b * T;
  for (int o = tid; o < owned; o += LOSS_THREADS) {
    int p = p0 + o;
    if (p >= 0 && p < T) g[p] = accumulate ? g[p] + tile[o] : tile[o];
  }
}

// ---------------------------------------------------------------------------------------------
// Backward, register-blocked (fft16.cuh): same block organisation as mss_bwd_kernel (a block owns the output frames
// whose first covering window lies in its range, recomputes every window that covers them, sums the covering
// windows per output frame in ascending order), but every transform keeps sixteen points per thread:
//   forward of window A  -> spectral gradient of A written into the REAL lane of a register spectrum Y, bins k and
//                           N - k side by side in the thread that holds both (Hermitian extension for free);
//   forward of window B  -> the same into the IMAGINARY lane of Y;
//   transposed network   -> Y goes back to the time domain straight from those registers and arrives as element
//                           tid + m N/16 per thread: window, store, done.
// Two shared-memory exchanges per transform instead of four round trips, no pass that builds or symmetrises the
// gradient spectrum in shared memory, two transform buffers instead of three.
// ---------------------------------------------------------------------------------------------
template <int N>
struct Bwd16Geom {
  static constexpr int TT = N / 16;
  static constexpr int NF = LOSS16_THREADS / TT;                   // window pairs per round
  static constexpr int WR = 2 * NF;                                // windows per round
  static constexpr int ROUNDS = WR >= 16 ? 1 : 16 / WR;            // at least 16 windows per block
  static constexpr int WB = WR * ROUNDS;                           // windows per block
};

// Gradient of the two loss terms with respect to the spectrum of the prediction, one {k, N - k} pair of bins of
// z = FFT(x1 + i x2).  hk = half the gradient at bin k; lane 0 adds (hk, conj hk) to (Yk, Yn), lane 1 adds i times that.
__device__ __forceinline__ void grad_pair(float2 zk, float2 zn, float c_lin, float c_log2, int lane, float2 &Yk,
                                          float2 &Yn) {
  const float ax = zk.x + zn.x, ay = zk.y - zn.y;     // 2 X1[k]
  const float bx = zk.y + zn.y, by = zn.x - zk.x;     // 2 X2[k]
  const float m1 = fast_sqrt(fmaf(ax, ax, ay * ay)), m2 = fast_sqrt(fmaf(bx, bx, by * by));   // 2 |X1|, 2 |X2|
  const float ld = __log2f(m1 + 2.0f * LOG_EPS) - __log2f(m2 + 2.0f * LOG_EPS);
  // d/d|X1| of |(|X1| - |X2|)| and of |log(|X1| + eps) - log(|X2| + eps)|, with |X1| = m1 / 2
  const float gm = c_lin * sgn(m1 - m2) + c_log2 * sgn(ld) / (m1 + 2.0f * LOG_EPS);
  const float sc = 0.5f * gm / fmaxf(m1, 2e-8f);      // hk = (gm / 2) * X1 / max(|X1|, 1e-8) = sc * (2 X1)
  const float hx = sc * ax, hy = sc * ay;
  if (lane == 0) {
    Yk.x += hx; Yk.y += hy;
    Yn.x += hx; Yn.y -= hy;
  } else {  // times i: (x, y) -> (-y, x)
    Yk.x -= hy; Yk.y += hx;
    Yn.x += hy; Yn.y += hx;
  }
}
// a bin that is its own partner (0 and N/2): X1 = Re z real, only the real part of the gradient counts
__device__ __forceinline__ void grad_self(float2 z, float c_lin, float c_log2, int lane, float2 &Y) {
  const float m1 = 2.0f * fabsf(z.x), m2 = 2.0f * fabsf(z.y);
  const float ld = __log2f(m1 + 2.0f * LOG_EPS) - __log2f(m2 + 2.0f * LOG_EPS);
  const float gm = c_lin * sgn(m1 - m2) + c_log2 * sgn(ld) / (m1 + 2.0f * LOG_EPS);
  const float gre = gm / fmaxf(0.5f * m1, 1e-8f) * z.x;
  if (lane == 0) Y.x += gre; else Y.y += gre;
}

// MINB: resident blocks per SM the registers are capped for (3: 168 registers, nothing spilled; 4: 128 registers,
// a few spilled words in the middle sizes; 5: 102 registers).  4 is the default: measured 0.315 / 0.498 / 3.53 ms
// at 16 / 32 / 256 voices against 0.336 / 0.550 / 3.91 ms for 3.
template <int N, int MINB>
__global__ void __launch_bounds__(LOSS16_THREADS, MINB)
mss_bwd16_kernel(const float *__restrict__ pred, const float *__restrict__ target, int B, int T, int hop, int H,
                 int S /* windows whose first-covered frames this block owns */, const float *__restrict__ window,
                 const float2 *__restrict__ tw, float c_lin, float c_log, int accumulate, float *__restrict__ grad) {
  using Gm = Bwd16Geom<N>;
  using Ge = dgfft16::Geo<N>;
  constexpr int TT = Gm::TT, NF = Gm::NF, WR = Gm::WR, RL = Ge::RL;
  extern __shared__ float2 sm2[];
  using Lay = dgfft16::LayoutFree;   // conflict-free exchange layouts (the windowed results below keep pad())
  constexpr int PN = Lay::template size<N>();
  float2 *bufa_all = sm2, *bufb_all = sm2 + NF * PN;
  float *tile = reinterpret_cast<float *>(sm2 + 2 * NF * PN);
  const int tid = threadIdx.x, f = tid / TT, lt = tid % TT;
  const int b = blockIdx.y;
  const int hA = blockIdx.x * S;
  const int p0 = (hA - 1) * hop + 1;          // first owned frame (may be negative for the first block)
  const int owned = S * hop;
  const float *x1 = pred + (size_t)b * T, *x2 = target + (size_t)b * T;
  float2 *bufa = bufa_all + f * PN, *bufb = bufb_all + f * PN;
  // d/dm of log(m + eps) in terms of the doubled magnitude m' = 2 m: 2 / (m' + 2 eps)
  const float c_log2 = 2.0f * c_log;
  const int hop_shift = (hop & (hop - 1)) == 0 ? __ffs(hop) - 1 : -1;
  for (int o = tid; o < owned; o += LOSS16_THREADS) tile[o] = 0.0f;
  const int E = (N - 1) / hop;
  const int nwin = min(S + E, H - hA);        // windows this block must visit
  for (int r0 = 0; r0 < nwin; r0 += WR) {
    const int hr0 = hA + r0;
    float2 Y[Ge::PAIRS][2][RL];
#pragma unroll
    for (int p = 0; p < Ge::PAIRS; ++p)
#pragma unroll
      for (int e = 0; e < 2; ++e)
#pragma unroll
        for (int t = 0; t < RL; ++t) Y[p][e][t] = make_float2(0.f, 0.f);
#pragma unroll 1
    for (int w = 0; w < 2; ++w) {
      const int h = hr0 + 2 * f + w;
      const bool valid = h < H && (h - hA) < nwin;
      const int t_base = h * hop - (N - 1);
      float2 x[16];
      if (valid && t_base >= 0) {
        const float *p1 = x1 + t_base + lt, *p2 = x2 + t_base + lt, *wp = window + lt;
#pragma unroll
        for (int m = 0; m < 16; ++m) {
          const float wv = __ldg(wp + m * TT);
          x[m] = make_float2(p1[m * TT] * wv, p2[m * TT] * wv);
        }
      } else {
#pragma unroll
        for (int m = 0; m < 16; ++m) {
          const int i = lt + m * TT, t = t_base + i;
          float2 v = make_float2(0.f, 0.f);
          if (valid && t >= 0) {
            const float wv = __ldg(&window[i]);
            v = make_float2(x1[t] * wv, x2[t] * wv);
          }
          x[m] = v;
        }
      }
      float2 z[Ge::PAIRS][2][RL];
      dgfft16::sync_transform<N>();   // the previous transform's last reads of the buffers are done
      dgfft16::fft16<N, false, Lay>(x, z, bufa, bufb, lt, tw);
      if (valid) {
#pragma unroll
        for (int p = 0; p < Ge::PAIRS; ++p) {
          if (p > 0 || lt != 0) {
#pragma unroll
            for (int t = 0; t < RL; ++t) grad_pair(z[p][0][t], z[p][1][RL - 1 - t], c_lin, c_log2, w, Y[p][0][t], Y[p][1][RL - 1 - t]);
          } else {
            // butterflies 0 and N/(2 RL): bins pair up inside each of them
            grad_self(z[0][0][0], c_lin, c_log2, w, Y[0][0][0]);
            grad_self(z[0][0][RL / 2], c_lin, c_log2, w, Y[0][0][RL / 2]);
#pragma unroll
            for (int t = 1; t < RL / 2; ++t) grad_pair(z[0][0][t], z[0][0][RL - t], c_lin, c_log2, w, Y[0][0][t], Y[0][0][RL - t]);
#pragma unroll
            for (int t = 0; t < RL / 2; ++t) grad_pair(z[0][1][t], z[0][1][RL - 1 - t], c_lin, c_log2, w, Y[0][1][t], Y[0][1][RL - 1 - t]);
          }
        }
      }
    }
    // back to the time domain: un-normalised, + sign (Sources/DGen/Emit+SpectralLoss.swift:577-649)
    float2 g[16];
    dgfft16::sync_transform<N>();
    dgfft16::fft16_T<N, true, Lay>(Y, g, bufa, bufb, lt, tw);
    // bufb is free: the transposed network's last read of it is behind a barrier every thread has passed
    {
      const float *wp = window + lt;
#pragma unroll
      for (int m = 0; m < 16; ++m) {
        const float wv = __ldg(wp + m * TT);
        bufb[pad(lt + m * TT)] = make_float2(g[m].x * wv, g[m].y * wv);
      }
    }
    __syncthreads();
    const float2 *res = bufb_all;
    // only the owned frames this round's windows reach: [first window's start, last window's end]
    const int h_last = min(min(hr0 + WR - 1, H - 1), hA + nwin - 1);
    const int f_lo = max(max(p0, hr0 * hop - (N - 1)), 0), f_hi = min(min(p0 + owned - 1, h_last * hop), T - 1);
    for (int p = f_lo + tid; p <= f_hi; p += LOSS16_THREADS) {
      const int o = p - p0;
      // covering windows: ceil(p / hop) .. floor((p + N - 1) / hop); a shift when the hop is a power of two
      const int hlo = max(hr0, hop_shift >= 0 ? (p + hop - 1) >> hop_shift : (p + hop - 1) / hop);
      const int hhi = min(h_last, hop_shift >= 0 ? (p + N - 1) >> hop_shift : (p + N - 1) / hop);
      float acc = tile[o];
      for (int h = hlo; h <= hhi; ++h) {
        int slot = h - hr0;
        float2 v = res[(slot >> 1) * PN + pad(p - (h * hop - (N - 1)))];
        acc += (slot & 1) ? v.y : v.x;
      }
      tile[o] = acc;
    }
    __syncthreads();
  }
  float *gout = grad + (size_t)b * T;
  for (int o = tid; o < owned; o += LOSS16_THREADS) {
    int p = p0 + o;
    if (p >= 0 && p < T) gout[p] = accumulate ? gout[p] + tile[o] : tile[o];
  }
}

template <int N, int MINB>
int32_t launch_bwd16(dgc_ctx *ctx, const dgc_mss_params *p, const float *pred, const float *target, int hop, int H,
                     float c_lin, float c_log, int accumulate, float *grad) {
  using Gm = Bwd16Geom<N>;
  const float *win = dgc_ctx_hann_sym(ctx, N);
  const float2 *tw = dgc_ctx_twiddles(ctx, N);
  if (!win || !tw) return DGC_ERR_OOM;
  const int E = (N - 1) / hop;
  const int S0 = Gm::WB - E;
  if (S0 < 1) return dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "hop %d too small for window %d", hop, N);
  auto smem_of = [&](int S_) {
    return (size_t)2 * Gm::NF * dgfft16::LayoutFree::size<N>() * sizeof(float2) + (size_t)S_ * hop * sizeof(float);
  };
  if (smem_of(S0) > 200 * 1024) return dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "backward tile does not fit shared memory");
  cudaError_t e = cudaFuncSetAttribute(mss_bwd16_kernel<N, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  if (e != cudaSuccess) return dgc_fail(ctx, DGC_ERR_CUDA, "mss_bwd smem opt-in: %s", cudaGetErrorString(e));
  cudaFuncSetAttribute(mss_bwd16_kernel<N, MINB>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  // windows owned per block: the choice that minimises (waves of resident blocks x rounds per block), see launch_bwd;
  // the summation order per output frame does not depend on it
  int S = S0;
  {
    const auto key = std::make_pair(std::make_pair(N, -hop * 8 - MINB), std::make_pair(H, p->B));   // (-hop: this kernel's own entries)
    auto it = ctx->mss_bwd_owned.find(key);
    if (it != ctx->mss_bwd_owned.end()) {
      S = it->second;
    } else {
      // A block visits S + E windows in rounds of WR.  Few voices leave a grid of S0-window blocks far below the
      // number of resident slots (160 blocks on 444 slots for 16 voices at N = 2048: 7 % of the warps active), so
      // smaller S -- more, shorter blocks, at the price of revisiting the E overlap windows more often -- are
      // candidates too; ties go to the larger S (less revisiting).
      long long best = -1;
      for (int cand = 1; cand <= S0 + 24 && cand <= H + E; ++cand) {
        const size_t sm = smem_of(cand);
        if (sm > 200 * 1024) break;
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mss_bwd16_kernel<N, MINB>, LOSS16_THREADS, sm) != cudaSuccess ||
            per_sm < 1)
          break;
        const long long blocks = (long long)dgc_div_up(H + 1, cand) * p->B, slots = (long long)per_sm * ctx->sm_count;
        const long long waves = (blocks + slots - 1) / slots;
        const long long cost = waves * dgc_div_up(cand + E, Gm::WR);
        if (best < 0 || cost <= best) {
          best = cost;
          S = cand;
        }
      }
      ctx->mss_bwd_owned[key] = S;
    }
  }
  const size_t smem = smem_of(S);
  // block j owns the frames whose first covering window is in [j S, (j+1) S).  The frames behind the last window
  // ((H-1) hop, T-1] are covered by no window at all -- their "first covering window" would be number H -- and must
  // still be written (zero, or left as accumulated): the grid spans window indices 0 .. H.
  mss_bwd16_kernel<N, MINB><<<dim3(dgc_div_up(H + 1, S), p->B), LOSS16_THREADS, smem, ctx->stream>>>(
      pred, target, p->B, p->T, hop, H, S, win, tw, c_lin, c_log, accumulate, grad);
  ctx->launches++;
  return dgc_check_launch(ctx, "mss_bwd16");
}

template <int N>
int32_t launch_bwd(dgc_ctx *ctx, const dgc_mss_params *p, const float *pred, const float *target, int hop, int H,
                   float c_lin, float c_log, int accumulate, float *grad) {
  using Gm = BwdGeom<N>;
  const float *win = dgc_ctx_hann_sym(ctx, N);
  const float2 *tw = dgc_ctx_twiddles(ctx, N);
  if (!win || !tw) return DGC_ERR_OOM;
  const int E = (N - 1) / hop;
  const int S0 = Gm::WB - E;
  if (S0 < 1) return dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "hop %d too small for window %d", hop, N);
  auto smem_of = [&](int S_) {
    return (size_t)3 * Gm::NF * padded(N) * sizeof(float2) + (size_t)S_ * hop * sizeof(float);
  };
  if (smem_of(S0) > 200 * 1024) return dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "backward tile does not fit shared memory");
  cudaError_t e = cudaFuncSetAttribute(mss_bwd_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  if (e != cudaSuccess) return dgc_fail(ctx, DGC_ERR_CUDA, "mss_bwd smem opt-in: %s", cudaGetErrorString(e));
  // the kernel lives on shared memory, not on L1: ask for the largest shared-memory carve-out so that as many
  // blocks as the tile size allows are resident
  cudaFuncSetAttribute(mss_bwd_kernel<N>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  // Windows owned per block.  A block visits S + E windows (E = the windows before its first owned one that still
  // cover its frames), so a larger S wastes less on that overlap, but what decides the time of a launch this small
  // is whether the grid fills WHOLE waves of resident blocks: 320 blocks on 296 slots run as long as 592.  Among
  // the S that keep the shared-memory tile within bounds, take the one with the least (waves x rounds per block);
  // the summation order per output frame (covering windows ascending) does not depend on S, nor do the bits of
  // the result.
  int S = S0;
  {
    const auto key = std::make_pair(std::make_pair(N, hop), std::make_pair(H, p->B));
    auto it = ctx->mss_bwd_owned.find(key);
    if (it != ctx->mss_bwd_owned.end()) {
      S = it->second;
    } else {
      long long best = -1;
      int per_sm0 = 0;
      for (int cand = S0; cand <= S0 + 24 && cand <= H + E; ++cand) {
        const size_t sm = smem_of(cand);
        if (sm > 200 * 1024) break;
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mss_bwd_kernel<N>, LOSS_THREADS, sm) != cudaSuccess ||
            per_sm < 1)
          break;
        if (cand == S0) per_sm0 = per_sm;
        if (per_sm < per_sm0) break;   // a larger tile must not cost resident blocks
        const long long blocks = (long long)dgc_div_up(H + 1, cand) * p->B, slots = (long long)per_sm * ctx->sm_count;
        const long long waves = (blocks + slots - 1) / slots;
        const long long cost = waves * dgc_div_up(cand + E, Gm::WR);
        if (best < 0 || cost < best) {
          best = cost;
          S = cand;
        }
      }
      ctx->mss_bwd_owned[key] = S;
    }
  }
  const size_t smem = smem_of(S);
  // block j owns the frames whose first covering window is in [j*S, (j+1)*S); frames up to T-1 have
  // first covering window <= H-1
  mss_bwd_kernel<N><<<dim3(dgc_div_up(H + 1, S), p->B), LOSS_THREADS, smem, ctx->stream>>>(
      pred, target, p->B, p->T, hop, H, S, win, tw, c_lin, c_log, accumulate, grad);
  ctx->launches++;
  return dgc_check_launch(ctx, "mss_bwd");
}

int32_t validate(dgc_ctx *ctx, const dgc_mss_params *p) {
  DGC_REQUIRE(ctx, p->B > 0 && p->T > 0, "B and T must be positive");
  DGC_REQUIRE(ctx, p->nscales > 0 && p->nscales <= DGC_MSS_MAX_SCALES, "nscales out of range");
  DGC_REQUIRE(ctx, p->hop_div >= 1, "hop_div must be >= 1");
  for (int s = 0; s < p->nscales; ++s)
    DGC_REQUIRE(ctx, dgc_is_pow2(p->sizes[s]) && p->sizes[s] >= 16 && p->sizes[s] <= 2048,
                "window sizes must be powers of two in 16..2048");
  return DGC_OK;
}

inline int hop_of(const dgc_mss_params *p, int s) {
  int hop = p->sizes[s] / p->hop_div;
  return hop < 1 ? 1 : hop;
}

}  // namespace

DGC_EXPORT uint64_t dgc_mss_partial_floats(const dgc_mss_params *p) {
  if (!p || p->B <= 0 || p->T <= 0 || p->nscales <= 0 || p->nscales > DGC_MSS_MAX_SCALES || p->hop_div < 1) return 0;
  uint64_t n = 0;
  for (int s = 0; s < p->nscales; ++s) {
    if (p->sizes[s] > p->T) continue;  // the reference skips windows longer than the render
    int hop = hop_of(p, s);
    n += 2ull * (uint64_t)dgc_div_up(p->T, hop) * p->B;
  }
  return n;
}

DGC_EXPORT int32_t dgc_mss_loss_fwd(dgc_ctx *ctx, const dgc_mss_params *p, const float *pred_dev,
                                    const float *target_dev, float *partial_dev, double *loss_dev) {
  return dgc_mss_loss_fwd_sum(ctx, p, pred_dev, nullptr, target_dev, partial_dev, loss_dev);
}

// prediction = pred_dev + pred_b_dev (pred_b_dev may be null): lets two synthesis branches that ran
// concurrently feed the loss without a pass that adds them
int32_t dgc_mss_loss_fwd_sum(dgc_ctx *ctx, const dgc_mss_params *p, const float *pred_dev, const float *pred_b_dev,
                             const float *target_dev, float *partial_dev, double *loss_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, p && pred_dev && target_dev && loss_dev, "null pointer");
  int32_t rc = validate(ctx, p);
  if (rc != DGC_OK) return rc;
  float *part = partial_dev ? partial_dev : dgc_ctx_scratch(ctx, dgc_mss_partial_floats(p) + 4);
  if (!part) return DGC_ERR_OOM;
  ReduceDesc d;
  d.nscales = 0;
  long long off = 0;
  int used = 0;
  for (int s = 0; s < p->nscales; ++s) {
    const int N = p->sizes[s];
    if (N > p->T) continue;
    ++used;
  }
  // partial layout and summation order follow the caller's scale order; the launch runs the usable
  // scales largest window first
  int order[DGC_MSS_MAX_SCALES], no = 0;
  long long off_of[DGC_MSS_MAX_SCALES];
  for (int s = 0; s < p->nscales; ++s) {
    const int N = p->sizes[s];
    if (N > p->T) continue;
    if (N < 16 || N > 2048 || (N & (N - 1))) return dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "window size %d", N);
    const int H = dgc_div_up(p->T, hop_of(p, s));
    order[no++] = s;
    off_of[s] = off;
    d.off[d.nscales] = off;
    d.cnt[d.nscales] = (long long)H * p->B;
    d.nscales++;
    off += 2ll * H * p->B;
  }
  std::stable_sort(order, order + no, [&](int x, int y) { return p->sizes[x] > p->sizes[y]; });
  // windows of 64 points and more run on the sixteen-points-per-thread kernel (128-thread blocks), the two smallest
  // sizes on the eight-points-per-thread one (256-thread blocks): two descriptors, at most two launches
  static const bool force_old = [] {
    const char *e = getenv("DGC_MSS_FWD");
    return e && strcmp(e, "r8") == 0;
  }();
  FwdDesc fd16, fd8;
  fd16.nscales = fd8.nscales = 0;
  int blocks16 = 0, blocks8 = 0;
  for (int i = 0; i < no; ++i) {
    const int s = order[i], N = p->sizes[s];
    const int hop = hop_of(p, s), H = dgc_div_up(p->T, hop);
    const bool wide = N >= 64 && !force_old;
    FwdDesc &fd = wide ? fd16 : fd8;
    int &blocks = wide ? blocks16 : blocks8;
    const int k = fd.nscales++;
    fd.N[k] = N;
    fd.hop[k] = hop;
    fd.H[k] = H;
    fd.window[k] = dgc_ctx_hann_sym(ctx, N);
    fd.tw[k] = dgc_ctx_twiddles(ctx, N);
    if (!fd.window[k] || !fd.tw[k]) return DGC_ERR_OOM;
    fd.lin[k] = part + off_of[s];
    fd.lg[k] = fd.lin[k] + (long long)H * p->B;
    fd.first_block[k] = blocks;
    blocks += wide ? dgc_div_up(H, LOSS16_THREADS / (N / 16)) * p->B : dgc_div_up(H, LOSS_THREADS / (N / 8));
    fd.first_block[k + 1] = blocks;
  }
  // resident blocks per SM are limited by shared memory (6 x 34 KB): ask for the largest carve-out
  static const bool carved = [] {
    cudaFuncSetAttribute(mss_fwd_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(mss_fwd_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(mss_fwd16_kernel<true, false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(mss_fwd16_kernel<false, false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(mss_fwd16_kernel<false, true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    return true;
  }();
  (void)carved;
  if (fd16.nscales > 0) {
    // DGC_MSS_TMA=1: the windows' sample runs are staged by tensor-map copies when the signals qualify (rows a
    // multiple of 16 bytes long and 16-byte aligned).  Measured slower than the per-thread loads (one window group per
    // block leaves nothing to overlap the copy with), so the per-thread loads are the default.
    static const bool tma_on = [] {
      const char *e = getenv("DGC_MSS_TMA");
      return e && strcmp(e, "1") == 0;
    }();
    CUtensorMap mp, mt;
    memset(&mp, 0, sizeof(mp));
    memset(&mt, 0, sizeof(mt));
    bool tma = tma_on && !pred_b_dev && p->hop_div >= 1;
    tma = tma && dgtma::make_map_2d(&mp, pred_dev, p->B, p->T, SPAN_BOX) && dgtma::make_map_2d(&mt, target_dev, p->B, p->T, SPAN_BOX);
    if (pred_b_dev)
      mss_fwd16_kernel<true, false><<<blocks16, LOSS16_THREADS, FWD16_SMEM_BYTES, ctx->stream>>>(
          pred_dev, pred_b_dev, target_dev, p->B, p->T, fd16, mp, mt, ctx->status_dev);
    else if (tma)
      mss_fwd16_kernel<false, true><<<blocks16, LOSS16_THREADS, 2 * padded(2048) * (int)sizeof(float2), ctx->stream>>>(
          pred_dev, nullptr, target_dev, p->B, p->T, fd16, mp, mt, ctx->status_dev);
    else
      mss_fwd16_kernel<false, false><<<blocks16, LOSS16_THREADS, FWD16_SMEM_BYTES, ctx->stream>>>(
          pred_dev, nullptr, target_dev, p->B, p->T, fd16, mp, mt, ctx->status_dev);
    DGC_LAUNCHED(ctx, tma ? "mss_fwd16_tma" : "mss_fwd16");
  }
  if (fd8.nscales > 0) {
    if (pred_b_dev)
      mss_fwd_kernel<true><<<dim3(blocks8, p->B), LOSS_THREADS, FWD_SMEM_BYTES, ctx->stream>>>(pred_dev, pred_b_dev,
                                                                                               target_dev, p->B, p->T, fd8);
    else
      mss_fwd_kernel<false><<<dim3(blocks8, p->B), LOSS_THREADS, FWD_SMEM_BYTES, ctx->stream>>>(pred_dev, nullptr,
                                                                                                target_dev, p->B, p->T, fd8);
    DGC_LAUNCHED(ctx, "mss_fwd");
  }
  // weights: (w / nscales) with nscales = number of usable windows, normalize:true divides by T
  // (Examples/HarmonicE2E/Trainer.swift:553-586, Sources/DGenLazy/Functions.swift:951-954);
  // the batched loss is the mean over voices (Emit+SpectralLoss.swift:937-938)
  const double den = (double)p->B * (double)(used > 0 ? used : 1) * (double)p->T;
  mss_reduce_kernel<<<RED_BLOCKS, RED_THREADS, 0, ctx->stream>>>(part, d, (double)p->w_lin / den, (double)p->w_log / den,
                                                                  ctx->loss_accum + 64, ctx->ticket_dev, loss_dev);
  DGC_LAUNCHED(ctx, "mss_reduce");
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_mss_loss_bwd(dgc_ctx *ctx, const dgc_mss_params *p, const float *pred_dev,
                                    const float *target_dev, float upstream, float *grad_pred_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, p && pred_dev && target_dev && grad_pred_dev, "null pointer");
  int32_t rc = validate(ctx, p);
  if (rc != DGC_OK) return rc;
  int used = 0;
  for (int s = 0; s < p->nscales; ++s)
    if (p->sizes[s] <= p->T) ++used;
  if (used == 0) {
    DGC_CUDA(ctx, cudaMemsetAsync(grad_pred_dev, 0, (size_t)p->B * p->T * sizeof(float), ctx->stream));
    return DGC_OK;
  }
  const double den = (double)p->B * (double)used * (double)p->T;
  const float c_lin = (float)((double)upstream * (double)p->w_lin / den);
  const float c_log = (float)((double)upstream * (double)p->w_log / den);
  int accumulate = 0;
  for (int s = 0; s < p->nscales; ++s) {
    const int N = p->sizes[s];
    if (N > p->T) continue;
    const int hop = hop_of(p, s), H = dgc_div_up(p->T, hop);
    static const bool bwd_old = [] {
      const char *e = getenv("DGC_MSS_BWD");
      return e && strcmp(e, "r8") == 0;
    }();
    // windows of 64 points and more run on the sixteen-points-per-thread kernel
    const bool wide = N >= 64 && !bwd_old;
    static const int bwd_minb = [] {
      const char *e = getenv("DGC_MSS_BWD_BLOCKS");
      return e ? atoi(e) : 4;
    }();
    switch (wide ? N : -N) {
#define CASE(NN) case -NN: rc = launch_bwd<NN>(ctx, p, pred_dev, target_dev, hop, H, c_lin, c_log, accumulate, grad_pred_dev); break;
      CASE(16) CASE(32) CASE(64) CASE(128) CASE(256) CASE(512) CASE(1024) CASE(2048)
#undef CASE
#define CASE(NN)                                                                                                          \
  case NN:                                                                                                                \
    rc = bwd_minb >= 5 ? launch_bwd16<NN, 5>(ctx, p, pred_dev, target_dev, hop, H, c_lin, c_log, accumulate, grad_pred_dev) \
       : bwd_minb == 4 ? launch_bwd16<NN, 4>(ctx, p, pred_dev, target_dev, hop, H, c_lin, c_log, accumulate, grad_pred_dev) \
                       : launch_bwd16<NN, 3>(ctx, p, pred_dev, target_dev, hop, H, c_lin, c_log, accumulate, grad_pred_dev); \
    break;
      CASE(64) CASE(128) CASE(256) CASE(512) CASE(1024) CASE(2048)
#undef CASE
      default: return dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "window size %d", N);
    }
    if (rc != DGC_OK) return rc;
    accumulate = 1;
  }
  return DGC_OK;
}
