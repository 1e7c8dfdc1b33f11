// Hop-gated spectral blocks: buffer -> FFT (magnitude or half spectrum), partitioned spectral
// multiply-accumulate, IFFT, overlap-add.
//
// The reference gates these on a hop counter inside a per-frame loop (bufferView ring write every
// frame, window gather + host FFT call when the counter reads 0, scatter-add into an output ring:
// Sources/DGen/HigherOps.swift:738-813, Sources/DGen/Emit+FFT.swift:6-62,
// Sources/DGen/Emit+PartitionedConvolution.swift:26-113).  All hop frames are known up front, so
// here every window is gathered straight from the contiguous signal and transformed in shared
// memory, batched over hops x voices; two real windows share one complex transform; overlap-add
// is a gather (each output frame sums the <= N/hop windows that cover it, oldest first, which is
// the order the reference's ring accumulates them).
#include "common.cuh"
#include "fft.cuh"

namespace {

using namespace dgfft;
constexpr int ST_THREADS = 256;

// Pair p of transform slot holds real sequences (2p, 2p+1) of one signal v as re / im.
// SRC 0: bufferView windows of x[v]: element i of hop frame h = x[h*hop - (N-1) + i] * window[i]
// SRC 1: zero-padded partitions of one IR: element i of partition h = ir[h*hop + i], i < hop
// SRC 2: overlap-add aligned frames of x[v]: element i of hop frame h = x[h*hop + i] * window[i]
//        (the adjoint of the overlap-add scatter, used by the backward pass)
// OUT 0: magnitudes [V][H][N/2+1]     OUT 1: half spectra float2 [V][H][N/2+1]
template <int N, int SRC, int OUT>
__global__ void __launch_bounds__(ST_THREADS)
stft_kernel(const float *__restrict__ x, int T, int hop, int H, const float *__restrict__ window,
            const float2 *__restrict__ tw, float *__restrict__ out) {
  constexpr int G = N / 8, NF = ST_THREADS / G, NB = N / 2 + 1, PN = padded(N);
  __shared__ float2 bufa[NF * PN];
  __shared__ float2 bufb[NF * PN];
  const int tid = threadIdx.x, f = tid / G, lt = tid % G;
  const int v = blockIdx.y;
  const int pair = blockIdx.x * NF + f;
  const int h0 = 2 * pair, h1 = h0 + 1;
  const float *xv = x + (size_t)v * T;
  float2 *a = bufa + f * PN, *bb = bufb + f * PN;
  float2 vin[8];   // a thread's loads (stride G) are its inputs of the first radix-8 stage: kept in registers
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    int i = lt + q * G;
    float w = (SRC != 1 && window) ? __ldg(&window[i]) : 1.0f;
    float2 val = make_float2(0.f, 0.f);
    if (SRC == 0) {
      int t0 = h0 * hop - (N - 1) + i, t1 = h1 * hop - (N - 1) + i;
      if (h0 < H && t0 >= 0 && t0 < T) val.x = xv[t0] * w;
      if (h1 < H && t1 >= 0 && t1 < T) val.y = xv[t1] * w;
    } else if (SRC == 1) {
      int t0 = h0 * hop + i, t1 = h1 * hop + i;
      if (h0 < H && i < hop && t0 < T) val.x = xv[t0];
      if (h1 < H && i < hop && t1 < T) val.y = xv[t1];
    } else {
      int t0 = h0 * hop + i, t1 = h1 * hop + i;
      if (h0 < H && t0 < T) val.x = xv[t0] * w;
      if (h1 < H && t1 < T) val.y = xv[t1] * w;
    }
    vin[q] = val;
  }
  float2 *z = fft_block_regs<N, false>(vin, a, bb, lt, tw);
  // bins 0..N/2 of both sequences
  for (int k = lt; k < NB; k += G) {
    float2 zk = z[pad(k)], zn = z[pad((N - k) & (N - 1))];
    float2 X0 = make_float2(0.5f * (zk.x + zn.x), 0.5f * (zk.y - zn.y));
    float2 X1 = make_float2(0.5f * (zk.y + zn.y), 0.5f * (zn.x - zk.x));
    if (OUT == 0) {
      if (h0 < H) out[((size_t)v * H + h0) * NB + k] = sqrtf(X0.x * X0.x + X0.y * X0.y);
      if (h1 < H) out[((size_t)v * H + h1) * NB + k] = sqrtf(X1.x * X1.x + X1.y * X1.y);
    } else {
      float2 *o = reinterpret_cast<float2 *>(out);
      if (h0 < H) o[((size_t)v * H + h0) * NB + k] = X0;
      if (h1 < H) o[((size_t)v * H + h1) * NB + k] = X1;
    }
  }
}

// Y[v][h][k] = sum_{j < K, j <= h} Hs[j][k] * X[v][h-j][k]   (partitioned spectral MAC, j = 0 first)
// Block: 32 bins x 8 hop groups; each thread carries HPT consecutive hops of one bin.
constexpr int MAC_BINS = 32, MAC_HPT = 4, MAC_HT = 8 * MAC_HPT;

__global__ void __launch_bounds__(256)
partconv_mac_kernel(const float2 *__restrict__ X, const float2 *__restrict__ Hs, int H, int K, int NB,
                    float2 *__restrict__ Y) {
  extern __shared__ float2 smem[];
  float2 *hs = smem;                          // [K][MAC_BINS]
  float2 *xs = smem + (size_t)K * MAC_BINS;   // [MAC_HT + K - 1][MAC_BINS], row r <-> hop hb - (K-1) + r
  const int kb = blockIdx.x * MAC_BINS, hb = blockIdx.y * MAC_HT, v = blockIdx.z;
  const int bin = threadIdx.x & 31, hg = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < K * MAC_BINS; i += 256) {
    int j = i / MAC_BINS, kk = i % MAC_BINS;
    hs[i] = (kb + kk < NB) ? Hs[(size_t)j * NB + kb + kk] : make_float2(0.f, 0.f);
  }
  const int rows = MAC_HT + K - 1;
  for (int i = threadIdx.x; i < rows * MAC_BINS; i += 256) {
    int r = i / MAC_BINS, kk = i % MAC_BINS;
    int h = hb - (K - 1) + r;
    xs[i] = (h >= 0 && h < H && kb + kk < NB) ? X[((size_t)v * H + h) * NB + kb + kk] : make_float2(0.f, 0.f);
  }
  __syncthreads();
  float2 acc[MAC_HPT];
#pragma unroll
  for (int u = 0; u < MAC_HPT; ++u) acc[u] = make_float2(0.f, 0.f);
  // hop h = hb + hg*HPT + u reads X row (h - j) -> r = (K-1) + hg*HPT + u - j
  const int rbase = (K - 1) + hg * MAC_HPT;
  float2 win[MAC_HPT];
#pragma unroll
  for (int u = 0; u < MAC_HPT - 1; ++u) win[u] = xs[(size_t)(rbase + u) * MAC_BINS + bin];
  // j = 0 uses rows rbase..rbase+HPT-1; as j grows the window slides down by one row
  win[MAC_HPT - 1] = xs[(size_t)(rbase + MAC_HPT - 1) * MAC_BINS + bin];
  for (int j = 0; j < K; ++j) {
    float2 hv = hs[(size_t)j * MAC_BINS + bin];
#pragma unroll
    for (int u = 0; u < MAC_HPT; ++u) {
      // (ar*br - ai*bi, ar*bi + ai*br) accumulated as the host MAC service does
      acc[u].x += win[u].x * hv.x - win[u].y * hv.y;
      acc[u].y += win[u].x * hv.y + win[u].y * hv.x;
    }
#pragma unroll
    for (int u = MAC_HPT - 1; u > 0; --u) win[u] = win[u - 1];
    int r = rbase - j - 1;
    win[0] = r >= 0 ? xs[(size_t)r * MAC_BINS + bin] : make_float2(0.f, 0.f);
  }
  if (kb + bin < NB) {
#pragma unroll
    for (int u = 0; u < MAC_HPT; ++u) {
      int h = hb + hg * MAC_HPT + u;
      if (h < H) Y[((size_t)v * H + h) * NB + kb + bin] = acc[u];
    }
  }
}

// frames[v][h][i] = Re(IFFT(Y[v][h]))[i] / N * window[i] * gain ; two hops per complex transform
template <int N>
__global__ void __launch_bounds__(ST_THREADS)
istft_kernel(const float2 *__restrict__ Y, int H, const float *__restrict__ window, const float2 *__restrict__ tw,
             float gain, float *__restrict__ frames) {
  constexpr int G = N / 8, NF = ST_THREADS / G, NB = N / 2 + 1, PN = padded(N);
  __shared__ float2 bufa[NF * PN];
  __shared__ float2 bufb[NF * PN];
  const int tid = threadIdx.x, f = tid / G, lt = tid % G;
  const int v = blockIdx.y, pair = blockIdx.x * NF + f;
  const int h0 = 2 * pair, h1 = h0 + 1;
  float2 *a = bufa + f * PN, *bb = bufb + f * PN;
  // z = Y0 + i*Y1 with Hermitian extension: Y[N-k] = conj(Y[k])
  float2 vin[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    int k = lt + q * G;
    int ks = k <= N / 2 ? k : N - k;
    float2 y0 = make_float2(0.f, 0.f), y1 = y0;
    if (h0 < H) y0 = Y[((size_t)v * H + h0) * NB + ks];
    if (h1 < H) y1 = Y[((size_t)v * H + h1) * NB + ks];
    if (k > N / 2) { y0.y = -y0.y; y1.y = -y1.y; }
    vin[q] = make_float2(y0.x - y1.y, y0.y + y1.x);
  }
  float2 *z = fft_block_regs<N, true>(vin, a, bb, lt, tw);
  const float invn = 1.0f / (float)N;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    int i = lt + q * G;
    float w = window ? __ldg(&window[i]) : 1.0f;
    float2 val = z[pad(i)];
    if (h0 < H) frames[((size_t)v * H + h0) * N + i] = ((val.x * invn) * w) * gain;
    if (h1 < H) frames[((size_t)v * H + h1) * N + i] = ((val.y * invn) * w) * gain;
  }
}

// out[v][t] (+)= sum over hops h with 0 <= t - h*hop - offset < N of frames[v][h][t - h*hop - offset],
// oldest first.  offset 0: the forward overlap-add; offset -(N-1): the adjoint of the bufferView gather.
__global__ void overlap_add_kernel(const float *__restrict__ frames, int T, int N, int hop, int H, int offset,
                                   int accumulate, float *__restrict__ out) {
  int t = blockIdx.x * blockDim.x + threadIdx.x, v = blockIdx.y;
  if (t >= T) return;
  int u = t - offset;            // frame h covers u in [h*hop, h*hop + N)
  int hmax = min(H - 1, u / hop);
  int hmin = u - N < 0 ? 0 : (u - N) / hop + 1;
  float acc = 0.0f;
  for (int h = hmin; h <= hmax; ++h) acc += frames[((size_t)v * H + h) * N + (u - h * hop)];
  size_t o = (size_t)v * T + t;
  out[o] = accumulate ? out[o] + acc : acc;
}

// V[v][m][k] = sum_{j < K, m + j < H} conj(Hs[j][k]) * U[v][m+j][k]: adjoint of the partitioned MAC
__global__ void __launch_bounds__(256)
partconv_mac_adj_kernel(const float2 *__restrict__ U, const float2 *__restrict__ Hs, int H, int K, int NB,
                        float2 *__restrict__ V) {
  extern __shared__ float2 smem[];
  float2 *hs = smem;                          // [K][MAC_BINS]
  float2 *us = smem + (size_t)K * MAC_BINS;   // [MAC_HT + K - 1][MAC_BINS], row r <-> hop hb + r
  const int kb = blockIdx.x * MAC_BINS, hb = blockIdx.y * MAC_HT, v = blockIdx.z;
  const int bin = threadIdx.x & 31, hg = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < K * MAC_BINS; i += 256) {
    int j = i / MAC_BINS, kk = i % MAC_BINS;
    hs[i] = (kb + kk < NB) ? Hs[(size_t)j * NB + kb + kk] : make_float2(0.f, 0.f);
  }
  const int rows = MAC_HT + K - 1;
  for (int i = threadIdx.x; i < rows * MAC_BINS; i += 256) {
    int r = i / MAC_BINS, kk = i % MAC_BINS;
    int h = hb + r;
    us[i] = (h < H && kb + kk < NB) ? U[((size_t)v * H + h) * NB + kb + kk] : make_float2(0.f, 0.f);
  }
  __syncthreads();
  float2 acc[MAC_HPT];
#pragma unroll
  for (int u = 0; u < MAC_HPT; ++u) acc[u] = make_float2(0.f, 0.f);
  const int rbase = hg * MAC_HPT;  // hop m = hb + rbase + u reads row rbase + u + j
  for (int j = 0; j < K; ++j) {
    float2 hv = hs[(size_t)j * MAC_BINS + bin];
#pragma unroll
    for (int u = 0; u < MAC_HPT; ++u) {
      float2 x = us[(size_t)(rbase + u + j) * MAC_BINS + bin];
      acc[u].x += x.x * hv.x + x.y * hv.y;   // conj(h) * x
      acc[u].y += x.y * hv.x - x.x * hv.y;
    }
  }
  if (kb + bin < NB) {
#pragma unroll
    for (int u = 0; u < MAC_HPT; ++u) {
      int m = hb + rbase + u;
      if (m < H) V[((size_t)v * H + m) * NB + kb + bin] = acc[u];
    }
  }
}

// G[k][bin] = sum_v sum_h conj(X[v][h-k][bin]) * U[v][h][bin]: gradient of the IR partition spectra.
// block = (32 bins, partition k); 8 thread groups split the (voice, hop) sum, combined in fixed order.
__global__ void __launch_bounds__(256)
partconv_ir_grad_kernel(const float2 *__restrict__ X, const float2 *__restrict__ U, int V, int H, int NB,
                        float2 *__restrict__ G) {
  __shared__ float2 red[8][33];
  const int bin = blockIdx.x * 32 + (threadIdx.x & 31), k = blockIdx.y, grp = threadIdx.x >> 5;
  float2 acc = make_float2(0.f, 0.f);
  if (bin < NB) {
    const int terms = V * (H - k);
    for (int i = grp; i < terms; i += 8) {
      int v = i / (H - k), h = k + (i - v * (H - k));
      float2 x = X[((size_t)v * H + (h - k)) * NB + bin], u = U[((size_t)v * H + h) * NB + bin];
      acc.x += x.x * u.x + x.y * u.y;
      acc.y += x.x * u.y - x.y * u.x;
    }
  }
  red[grp][threadIdx.x & 31] = acc;
  __syncthreads();
  if (grp == 0 && bin < NB) {
    float2 t = make_float2(0.f, 0.f);
#pragma unroll
    for (int g2 = 0; g2 < 8; ++g2) {
      t.x += red[g2][threadIdx.x & 31].x;
      t.y += red[g2][threadIdx.x & 31].y;
    }
    G[(size_t)k * NB + bin] = t;
  }
}

// g_ir[k*hop + i] = frames[k][i], i < hop (the zero-padded tail of each partition carries no parameter)
__global__ void take_partitions_kernel(const float *__restrict__ frames, int ir_len, int N, int hop,
                                       float *__restrict__ g_ir) {
  int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= ir_len) return;
  int k = t / hop, i = t - k * hop;
  g_ir[t] = frames[(size_t)k * N + i];
}

// half spectra float2 [rows][N/2+1] -> all N bins as split re / im [rows][N] (bins above N/2: the conjugate mirror,
// which is what a complex transform of a real window holds there)
__global__ void half_to_full_kernel(const float2 *__restrict__ half, int64_t rows, int N, float *__restrict__ re,
                                    float *__restrict__ im) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * N) return;
  const int64_t r = idx / N;
  const int k = (int)(idx - r * N), NB = N / 2 + 1;
  const float2 z = half[r * NB + (k <= N / 2 ? k : N - k)];
  re[idx] = z.x;
  im[idx] = k <= N / 2 ? z.y : -z.y;
}

// split re / im [rows][N] of ANY complex spectrum -> the half spectrum of its Hermitian part, whose inverse
// transform is the real part of the inverse transform of the whole (the reference keeps only that real part)
__global__ void full_to_half_kernel(const float *__restrict__ re, const float *__restrict__ im, int64_t rows, int N,
                                    float2 *__restrict__ half) {
  const int NB = N / 2 + 1;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * NB) return;
  const int64_t r = idx / NB;
  const int k = (int)(idx - r * NB), kn = (N - k) & (N - 1);
  const float *rr = re + r * N, *ii = im + r * N;
  half[idx] = make_float2(0.5f * (rr[k] + rr[kn]), 0.5f * (ii[k] - ii[kn]));
}

template <int N, int SRC, int OUT>
int32_t launch_stft(dgc_ctx *ctx, const float *x, int V, int T, int hop, int H, const float *window, float *out) {
  const float2 *tw = dgc_ctx_twiddles(ctx, N);
  if (!tw) return DGC_ERR_OOM;
  constexpr int NF = ST_THREADS / (N / 8);
  int pairs = (H + 1) / 2;
  stft_kernel<N, SRC, OUT><<<dim3(dgc_div_up(pairs, NF), V), ST_THREADS, 0, ctx->stream>>>(x, T, hop, H, window, tw,
                                                                                          out);
  ctx->launches++;
  return dgc_check_launch(ctx, "stft");
}

template <int SRC, int OUT>
int32_t dispatch_stft(dgc_ctx *ctx, int N, const float *x, int V, int T, int hop, int H, const float *window,
                      float *out) {
  switch (N) {
#define CASE(NN) case NN: return launch_stft<NN, SRC, OUT>(ctx, x, V, T, hop, H, window, out);
    CASE(16) CASE(32) CASE(64) CASE(128) CASE(256) CASE(512) CASE(1024) CASE(2048)
#undef CASE
  }
  return dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "FFT size %d (powers of two 16..2048)", N);
}

template <int N>
int32_t launch_istft(dgc_ctx *ctx, const float2 *Y, int V, int H, const float *window, float gain, float *frames) {
  const float2 *tw = dgc_ctx_twiddles(ctx, N);
  if (!tw) return DGC_ERR_OOM;
  constexpr int NF = ST_THREADS / (N / 8);
  int pairs = (H + 1) / 2;
  istft_kernel<N><<<dim3(dgc_div_up(pairs, NF), V), ST_THREADS, 0, ctx->stream>>>(Y, H, window, tw, gain, frames);
  ctx->launches++;
  return dgc_check_launch(ctx, "istft");
}

}  // namespace

DGC_EXPORT int32_t dgc_stft_mag(dgc_ctx *ctx, const float *x_dev, int32_t V, int32_t T, int32_t N, int32_t hop,
                                const float *window_dev, float *mags_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, x_dev && mags_dev, "null pointer");
  DGC_REQUIRE(ctx, V > 0 && V <= 65535 && T > 0 && hop > 0, "size out of range");
  DGC_REQUIRE(ctx, dgc_is_pow2(N) && N >= 16 && N <= 2048, "N must be a power of two in 16..2048");
  const int H = dgc_div_up(T, hop);
  return dispatch_stft<0, 0>(ctx, N, x_dev, V, T, hop, H, window_dev, mags_dev);
}

DGC_EXPORT uint64_t dgc_stft_scratch_floats(int32_t V, int32_t T, int32_t N, int32_t hop, int32_t inverse) {
  if (V <= 0 || T <= 0 || N <= 0 || hop <= 0) return 0;
  const uint64_t H = (uint64_t)(T + hop - 1) / hop, NB = N / 2 + 1;
  return ((2 * (uint64_t)V * H * NB + 3) & ~3ull) + (inverse ? (uint64_t)V * H * N : 0) + 16;
}

DGC_EXPORT int32_t dgc_stft_fwd(dgc_ctx *ctx, const float *x_dev, int32_t V, int32_t T, int32_t N, int32_t hop,
                                const float *window_dev, float *scratch_dev, float *re_dev, float *im_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, x_dev && re_dev && im_dev, "null pointer");
  DGC_REQUIRE(ctx, V > 0 && V <= 65535 && T > 0 && hop > 0, "size out of range");
  DGC_REQUIRE(ctx, dgc_is_pow2(N) && N >= 16 && N <= 2048, "N must be a power of two in 16..2048");
  const int H = dgc_div_up(T, hop);
  float *scr = scratch_dev ? scratch_dev : dgc_ctx_scratch(ctx, dgc_stft_scratch_floats(V, T, N, hop, 0));
  if (!scr) return DGC_ERR_OOM;
  DGC_REQUIRE(ctx, (((uintptr_t)scr) & 7) == 0, "scratch must be 8-byte aligned");
  int32_t rc = dispatch_stft<0, 1>(ctx, N, x_dev, V, T, hop, H, window_dev, scr);
  if (rc != DGC_OK) return rc;
  const int64_t rows = (int64_t)V * H;
  half_to_full_kernel<<<dgc_div_up(rows * N, 256), 256, 0, ctx->stream>>>(reinterpret_cast<const float2 *>(scr), rows, N,
                                                                         re_dev, im_dev);
  DGC_LAUNCHED(ctx, "stft_full_bins");
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_istft_ola(dgc_ctx *ctx, const float *re_dev, const float *im_dev, int32_t V, int32_t T, int32_t N,
                                 int32_t hop, const float *window_dev, float gain, float *scratch_dev,
                                 int32_t accumulate, float *out_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, re_dev && im_dev && out_dev, "null pointer");
  DGC_REQUIRE(ctx, V > 0 && V <= 65535 && T > 0, "size out of range");
  DGC_REQUIRE(ctx, dgc_is_pow2(N) && N >= 16 && N <= 2048, "N must be a power of two in 16..2048");
  DGC_REQUIRE(ctx, hop > 0 && hop <= N, "hop must be in 1..N");
  const int H = dgc_div_up(T, hop), NB = N / 2 + 1;
  float *scr = scratch_dev ? scratch_dev : dgc_ctx_scratch(ctx, dgc_stft_scratch_floats(V, T, N, hop, 1));
  if (!scr) return DGC_ERR_OOM;
  DGC_REQUIRE(ctx, (((uintptr_t)scr) & 7) == 0, "scratch must be 8-byte aligned");
  float *frames = scr + (((size_t)2 * V * H * NB + 3) & ~(size_t)3);
  const int64_t rows = (int64_t)V * H;
  full_to_half_kernel<<<dgc_div_up(rows * NB, 256), 256, 0, ctx->stream>>>(re_dev, im_dev, rows, N,
                                                                          reinterpret_cast<float2 *>(scr));
  DGC_LAUNCHED(ctx, "istft_hermitian_part");
  int32_t rc = DGC_OK;
  switch (N) {
#define CASE(NN) case NN: rc = launch_istft<NN>(ctx, reinterpret_cast<const float2 *>(scr), V, H, window_dev, gain, frames); break;
    CASE(16) CASE(32) CASE(64) CASE(128) CASE(256) CASE(512) CASE(1024) CASE(2048)
#undef CASE
  }
  if (rc != DGC_OK) return rc;
  overlap_add_kernel<<<dim3(dgc_div_up(T, 256), V), 256, 0, ctx->stream>>>(frames, T, N, hop, H, 0, accumulate,
                                                                           out_dev);
  DGC_LAUNCHED(ctx, "overlap_add");
  return DGC_OK;
}

DGC_EXPORT uint64_t dgc_partconv_scratch_floats(int32_t V, int32_t T, int32_t ir_len, int32_t N, int32_t hop) {
  if (V <= 0 || T <= 0 || ir_len <= 0 || N <= 0 || hop <= 0) return 0;
  uint64_t H = (uint64_t)(T + hop - 1) / hop, K = (uint64_t)(ir_len + hop - 1) / hop, NB = N / 2 + 1;
  // IR spectra, X spectra, Y spectra (float2 each), frames
  return 2 * K * NB + 2 * (uint64_t)V * H * NB * 2 + (uint64_t)V * H * N + 64;
}

DGC_EXPORT int32_t dgc_partconv(dgc_ctx *ctx, const float *x_dev, int32_t V, int32_t T, const float *ir_dev,
                                int32_t ir_len, int32_t N, int32_t hop, float gain, float *scratch_dev,
                                int32_t accumulate, float *out_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, x_dev && ir_dev && out_dev, "null pointer");
  DGC_REQUIRE(ctx, V > 0 && V <= 65535 && T > 0 && ir_len > 0, "size out of range");
  DGC_REQUIRE(ctx, dgc_is_pow2(N) && N >= 16 && N <= 2048, "N must be a power of two in 16..2048");
  DGC_REQUIRE(ctx, hop > 0 && hop <= N, "hop must be in 1..N");
  const int H = dgc_div_up(T, hop), K = dgc_div_up(ir_len, hop), NB = N / 2 + 1;
  size_t mac_smem = ((size_t)K * MAC_BINS + (size_t)(MAC_HT + K - 1) * MAC_BINS) * sizeof(float2);
  DGC_REQUIRE(ctx, mac_smem <= 200 * 1024, "impulse response has too many partitions (K <= 380)");
  DGC_REQUIRE(ctx, dgc_div_up(H, MAC_HT) <= 65535, "too many hops");
  float *scr = scratch_dev ? scratch_dev : dgc_ctx_scratch(ctx, dgc_partconv_scratch_floats(V, T, ir_len, N, hop));
  if (!scr) return DGC_ERR_OOM;
  DGC_REQUIRE(ctx, (((uintptr_t)scr) & 15) == 0, "scratch must be 16-byte aligned");
  float *hs = scr;
  float *xs = hs + (((size_t)2 * K * NB + 3) & ~(size_t)3);
  float *ys = xs + (((size_t)2 * V * H * NB + 3) & ~(size_t)3);
  float *frames = ys + (((size_t)2 * V * H * NB + 3) & ~(size_t)3);
  const float *win = dgc_ctx_hann_per(ctx, N);
  if (!win) return DGC_ERR_OOM;
  // partitionIR: FFT of each zero-padded partition (Sources/DGenLazy/SpectralTensorOps.swift:219-243)
  int32_t rc = dispatch_stft<1, 1>(ctx, N, ir_dev, 1, ir_len, hop, K, nullptr, hs);
  if (rc != DGC_OK) return rc;
  // X_h = FFT(hann * window_h)
  rc = dispatch_stft<0, 1>(ctx, N, x_dev, V, T, hop, H, win, xs);
  if (rc != DGC_OK) return rc;
  DGC_CUDA(ctx, cudaFuncSetAttribute(partconv_mac_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mac_smem));
  partconv_mac_kernel<<<dim3(dgc_div_up(NB, MAC_BINS), dgc_div_up(H, MAC_HT), V), 256, mac_smem, ctx->stream>>>(
      reinterpret_cast<const float2 *>(xs), reinterpret_cast<const float2 *>(hs), H, K, NB,
      reinterpret_cast<float2 *>(ys));
  DGC_LAUNCHED(ctx, "partconv_mac");
  switch (N) {
#define CASE(NN) case NN: rc = launch_istft<NN>(ctx, reinterpret_cast<const float2 *>(ys), V, H, win, gain, frames); break;
    CASE(16) CASE(32) CASE(64) CASE(128) CASE(256) CASE(512) CASE(1024) CASE(2048)
#undef CASE
  }
  if (rc != DGC_OK) return rc;
  overlap_add_kernel<<<dim3(dgc_div_up(T, 256), V), 256, 0, ctx->stream>>>(frames, T, N, hop, H, 0, accumulate,
                                                                           out_dev);
  DGC_LAUNCHED(ctx, "overlap_add");
  return DGC_OK;
}

DGC_EXPORT uint64_t dgc_partconv_bwd_scratch_floats(int32_t V, int32_t T, int32_t ir_len, int32_t N, int32_t hop) {
  if (V <= 0 || T <= 0 || ir_len <= 0 || N <= 0 || hop <= 0) return 0;
  uint64_t H = (uint64_t)(T + hop - 1) / hop, K = (uint64_t)(ir_len + hop - 1) / hop, NB = N / 2 + 1;
  // IR spectra + IR-gradient spectra, X, U, V spectra, frames (max of V*H and K frames)
  uint64_t fr = (uint64_t)V * H > K ? (uint64_t)V * H : K;
  return 4 * K * NB + 3 * (2 * (uint64_t)V * H * NB + 4) + fr * N + 64;
}

// Backward of dgc_partconv (a linear map in x and in ir): g_x = A(ir)^T g_out and/or g_ir.  The reference
// has no backward for partitionedSpectralConvolve (Sources/DGen/Gradients.swift:1156-1164); this is the
// exact adjoint of the forward above, checked against an fp64 evaluation.
DGC_EXPORT int32_t dgc_partconv_bwd(dgc_ctx *ctx, const float *x_dev, int32_t V, int32_t T, const float *ir_dev,
                                    int32_t ir_len, int32_t N, int32_t hop, float gain, const float *g_out_dev,
                                    float *scratch_dev, int32_t accumulate_gx, float *g_x_dev, float *g_ir_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, x_dev && ir_dev && g_out_dev && (g_x_dev || g_ir_dev), "null pointer");
  DGC_REQUIRE(ctx, V > 0 && V <= 65535 && T > 0 && ir_len > 0, "size out of range");
  DGC_REQUIRE(ctx, dgc_is_pow2(N) && N >= 16 && N <= 2048, "N must be a power of two in 16..2048");
  DGC_REQUIRE(ctx, hop > 0 && hop <= N, "hop must be in 1..N");
  const int H = dgc_div_up(T, hop), K = dgc_div_up(ir_len, hop), NB = N / 2 + 1;
  size_t mac_smem = ((size_t)K * MAC_BINS + (size_t)(MAC_HT + K - 1) * MAC_BINS) * sizeof(float2);
  DGC_REQUIRE(ctx, mac_smem <= 200 * 1024, "impulse response has too many partitions (K <= 380)");
  float *scr = scratch_dev ? scratch_dev
                           : dgc_ctx_scratch(ctx, dgc_partconv_bwd_scratch_floats(V, T, ir_len, N, hop));
  if (!scr) return DGC_ERR_OOM;
  DGC_REQUIRE(ctx, (((uintptr_t)scr) & 15) == 0, "scratch must be 16-byte aligned");
  const size_t nh = ((size_t)2 * K * NB + 3) & ~(size_t)3, nx = ((size_t)2 * V * H * NB + 3) & ~(size_t)3;
  float *hs = scr, *gs = hs + nh, *xs = gs + nh, *us = xs + nx, *vs = us + nx, *frames = vs + nx;
  const float *win = dgc_ctx_hann_per(ctx, N);
  if (!win) return DGC_ERR_OOM;
  int32_t rc = dispatch_stft<2, 1>(ctx, N, g_out_dev, V, T, hop, H, win, us);   // U_h = FFT(w * g[h*hop ..])
  if (rc != DGC_OK) return rc;
  if (g_x_dev) {
    rc = dispatch_stft<1, 1>(ctx, N, ir_dev, 1, ir_len, hop, K, nullptr, hs);
    if (rc != DGC_OK) return rc;
    DGC_CUDA(ctx, cudaFuncSetAttribute(partconv_mac_adj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)mac_smem));
    partconv_mac_adj_kernel<<<dim3(dgc_div_up(NB, MAC_BINS), dgc_div_up(H, MAC_HT), V), 256, mac_smem, ctx->stream>>>(
        reinterpret_cast<const float2 *>(us), reinterpret_cast<const float2 *>(hs), H, K, NB,
        reinterpret_cast<float2 *>(vs));
    DGC_LAUNCHED(ctx, "partconv_mac_adj");
    switch (N) {
#define CASE(NN) case NN: rc = launch_istft<NN>(ctx, reinterpret_cast<const float2 *>(vs), V, H, win, gain, frames); break;
      CASE(16) CASE(32) CASE(64) CASE(128) CASE(256) CASE(512) CASE(1024) CASE(2048)
#undef CASE
    }
    if (rc != DGC_OK) return rc;
    overlap_add_kernel<<<dim3(dgc_div_up(T, 256), V), 256, 0, ctx->stream>>>(frames, T, N, hop, H, -(N - 1),
                                                                             accumulate_gx, g_x_dev);
    DGC_LAUNCHED(ctx, "overlap_add_adj");
  }
  if (g_ir_dev) {
    rc = dispatch_stft<0, 1>(ctx, N, x_dev, V, T, hop, H, win, xs);
    if (rc != DGC_OK) return rc;
    partconv_ir_grad_kernel<<<dim3(dgc_div_up(NB, 32), K), 256, 0, ctx->stream>>>(
        reinterpret_cast<const float2 *>(xs), reinterpret_cast<const float2 *>(us), V, H, NB,
        reinterpret_cast<float2 *>(gs));
    DGC_LAUNCHED(ctx, "partconv_ir_grad");
    switch (N) {
#define CASE(NN) case NN: rc = launch_istft<NN>(ctx, reinterpret_cast<const float2 *>(gs), 1, K, nullptr, gain, frames); break;
      CASE(16) CASE(32) CASE(64) CASE(128) CASE(256) CASE(512) CASE(1024) CASE(2048)
#undef CASE
    }
    if (rc != DGC_OK) return rc;
    take_partitions_kernel<<<dgc_div_up(ir_len, 256), 256, 0, ctx->stream>>>(frames, ir_len, N, hop, g_ir_dev);
    DGC_LAUNCHED(ctx, "take_partitions");
  }
  return DGC_OK;
}
