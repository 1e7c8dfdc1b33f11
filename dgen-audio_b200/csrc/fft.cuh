// Shared-memory Stockham FFT building blocks (radix 8 / 4 / 2), used by the spectral loss, the
// STFT and the partitioned convolution.  A transform of N points is carried by N/8 threads; each
// stage reads N points from one shared buffer, applies twiddles and a radix-R butterfly in
// registers, and writes to the other buffer in the self-sorting (Stockham) order, so no bit
// reversal pass exists.  Convention: forward X[k] = sum x[n] exp(-2 pi i k n / N), unnormalised in
// both directions (the host FFT service of the reference, Sources/DGenHostSupport/DGenHostSupport.c:10-30).
#pragma once
#include <cuda_runtime.h>

namespace dgfft {

// Shared-memory index padding: one extra float2 after every 16, so that the power-of-two strides of the
// Stockham scatter (stride R after the first stage) spread over all banks.  Every access to a transform
// buffer goes through pad(); a buffer of N points occupies padded(N) float2.
__host__ __device__ constexpr int padded(int n) { return n + (n >> 4); }
__device__ __forceinline__ int pad(int i) { return i + (i >> 4); }

__device__ __forceinline__ float2 cmul(float2 a, float2 b) {
  return make_float2(fmaf(a.x, b.x, -a.y * b.y), fmaf(a.x, b.y, a.y * b.x));
}
__device__ __forceinline__ float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 csub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
// multiply by -i (forward) or +i (inverse)
template <bool INV>
__device__ __forceinline__ float2 rot90(float2 a) {
  return INV ? make_float2(-a.y, a.x) : make_float2(a.y, -a.x);
}

template <bool INV>
__device__ __forceinline__ void dft2(float2 &a, float2 &b) {
  float2 t = a;
  a = cadd(t, b);
  b = csub(t, b);
}

template <bool INV>
__device__ __forceinline__ void dft4(float2 &a, float2 &b, float2 &c, float2 &d) {
  float2 s0 = cadd(a, c), s1 = csub(a, c), s2 = cadd(b, d), s3 = rot90<INV>(csub(b, d));
  a = cadd(s0, s2);
  b = cadd(s1, s3);
  c = csub(s0, s2);
  d = csub(s1, s3);
}

template <bool INV>
__device__ __forceinline__ void dft8(float2 *v) {
  // even / odd radix-4, then combine with W8^k
  dft4<INV>(v[0], v[2], v[4], v[6]);
  dft4<INV>(v[1], v[3], v[5], v[7]);
  const float h = 0.70710678118654752f;
  float2 o1 = v[3], o2 = v[5], o3 = v[7];
  // W8^1 = h(1 -+ i), W8^2 = -+ i, W8^3 = h(-1 -+ i)
  float2 w1 = INV ? make_float2(h * (o1.x - o1.y), h * (o1.x + o1.y)) : make_float2(h * (o1.x + o1.y), h * (o1.y - o1.x));
  float2 w2 = rot90<INV>(o2);
  float2 w3 = INV ? make_float2(-h * (o3.x + o3.y), h * (o3.x - o3.y)) : make_float2(h * (o3.y - o3.x), -h * (o3.x + o3.y));
  float2 e0 = v[0], e1 = v[2], e2 = v[4], e3 = v[6], o0 = v[1];
  v[0] = cadd(e0, o0); v[4] = csub(e0, o0);
  v[1] = cadd(e1, w1); v[5] = csub(e1, w1);
  v[2] = cadd(e2, w2); v[6] = csub(e2, w2);
  v[3] = cadd(e3, w3); v[7] = csub(e3, w3);
}

template <int R, bool INV>
__device__ __forceinline__ void dftR(float2 *v) {
  if (R == 8) dft8<INV>(v);
  else if (R == 4) dft4<INV>(v[0], v[1], v[2], v[3]);
  else dft2<INV>(v[0], v[1]);
}

// One Stockham stage of radix R with input stride Ns (product of the radices already applied).
// tid in [0, N/8); tw is the table exp(-2 pi i m / N), m < N.
template <int N, int R, bool INV>
__device__ __forceinline__ void stage(const float2 *__restrict__ in, float2 *__restrict__ out, int Ns, int tid,
                                      const float2 *__restrict__ tw) {
  constexpr int PER = 8 / R;
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    const int j = tid + q * (N / 8);
    const int k = j & (Ns - 1);
    float2 v[R];
#pragma unroll
    for (int t = 0; t < R; ++t) v[t] = in[pad(j + t * (N / R))];
    if (Ns > 1) {
      const int step = N / (Ns * R);
      if (R == 8) {
        // w^1, w^2, w^4 from the table, the other four powers as products of those (one rounding more than a
        // table value): three loads per butterfly instead of seven on the load/store pipe the stage is bound by
        float2 w1 = __ldg(&tw[k * step]), w2 = __ldg(&tw[k * 2 * step]), w4 = __ldg(&tw[k * 4 * step]);
        if (INV) { w1.y = -w1.y; w2.y = -w2.y; w4.y = -w4.y; }
        const float2 w3 = cmul(w1, w2), w5 = cmul(w1, w4), w6 = cmul(w2, w4), w7 = cmul(w3, w4);
        v[1] = cmul(v[1], w1); v[2] = cmul(v[2], w2); v[3] = cmul(v[3], w3); v[4] = cmul(v[4], w4);
        v[5] = cmul(v[5], w5); v[6] = cmul(v[6], w6); v[7] = cmul(v[7], w7);
      } else {
#pragma unroll
        for (int t = 1; t < R; ++t) {
          float2 w = __ldg(&tw[k * t * step]);
          if (INV) w.y = -w.y;
          v[t] = cmul(v[t], w);
        }
      }
    }
    dftR<R, INV>(v);
    const int j0 = (j - k) * R + k;
#pragma unroll
    for (int t = 0; t < R; ++t) out[pad(j0 + t * Ns)] = v[t];
  }
}

// Full transform of N points held in shared buffer `a` (scratch buffer `b`); N/8 threads take part
// and every thread of the block must call this.  Between stages it synchronises the threads that share the
// transform: the whole block when a transform spans several warps, only the warp when its N/8 <= 32 threads sit
// inside one (transforms of other warps touch other buffers).  Callers that let OTHER threads read the result
// synchronise the block themselves.  Returns the buffer that holds the result in natural order.
template <int N>
__device__ __forceinline__ void fft_sync() {
  if (N / 8 <= 32) __syncwarp();
  else __syncthreads();
}

template <int N, bool INV>
__device__ __forceinline__ float2 *fft_block(float2 *a, float2 *b, int tid, const float2 *__restrict__ tw) {
  static_assert(N >= 16 && N <= 4096 && (N & (N - 1)) == 0, "N must be a power of two in 16..4096");
  int Ns = 1;
  float2 *src = a, *dst = b, *t;
  constexpr int LOG = N == 16 ? 4 : N == 32 ? 5 : N == 64 ? 6 : N == 128 ? 7 : N == 256 ? 8 : N == 512 ? 9
                      : N == 1024 ? 10 : N == 2048 ? 11 : 12;
  constexpr int N8 = LOG / 3, REM = LOG % 3;
#pragma unroll
  for (int s = 0; s < N8; ++s) {
    stage<N, 8, INV>(src, dst, Ns, tid, tw);
    Ns *= 8;
    t = src; src = dst; dst = t;
    fft_sync<N>();
  }
  if (REM == 2) {
    stage<N, 4, INV>(src, dst, Ns, tid, tw);
    t = src; src = dst; dst = t;
    fft_sync<N>();
  } else if (REM == 1) {
    stage<N, 2, INV>(src, dst, Ns, tid, tw);
    t = src; src = dst; dst = t;
    fft_sync<N>();
  }
  return src;
}

// The same transform when thread `tid` already HOLDS its eight inputs of the first stage in registers
// (v[t] = element tid + t * N/8, which is exactly what a thread that fills the buffer with stride N/8 produces):
// the first radix-8 stage runs straight from the registers, which saves writing the inputs to shared memory,
// the barrier after that, and reading them back.  `a` receives the first stage's output; nobody may still be
// reading `a` or `b` when this is called.
template <int N, bool INV>
__device__ __forceinline__ float2 *fft_block_regs(float2 (&v)[8], float2 *a, float2 *b, int tid,
                                                  const float2 *__restrict__ tw) {
  static_assert(N >= 16 && N <= 4096 && (N & (N - 1)) == 0, "N must be a power of two in 16..4096");
  constexpr int LOG = N == 16 ? 4 : N == 32 ? 5 : N == 64 ? 6 : N == 128 ? 7 : N == 256 ? 8 : N == 512 ? 9
                      : N == 1024 ? 10 : N == 2048 ? 11 : 12;
  constexpr int N8 = LOG / 3, REM = LOG % 3;
  dft8<INV>(v);
#pragma unroll
  for (int t = 0; t < 8; ++t) a[pad(tid * 8 + t)] = v[t];
  fft_sync<N>();
  int Ns = 8;
  float2 *src = a, *dst = b, *t;
#pragma unroll
  for (int s = 1; s < N8; ++s) {
    stage<N, 8, INV>(src, dst, Ns, tid, tw);
    Ns *= 8;
    t = src; src = dst; dst = t;
    fft_sync<N>();
  }
  if (REM == 2) {
    stage<N, 4, INV>(src, dst, Ns, tid, tw);
    t = src; src = dst; dst = t;
    fft_sync<N>();
  } else if (REM == 1) {
    stage<N, 2, INV>(src, dst, Ns, tid, tw);
    t = src; src = dst; dst = t;
    fft_sync<N>();
  }
  return src;
}

}  // namespace dgfft
