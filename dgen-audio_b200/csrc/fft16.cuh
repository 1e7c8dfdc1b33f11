// Register-blocked Stockham FFT: sixteen complex points per thread, N/16 threads per transform.
//
// The transforms of fft.cuh keep eight points per thread and exchange through shared memory after every radix-8
// stage; for N = 2048 that is four trips through the shared-memory pipe (three exchanges plus the read of the
// result), and that pipe, not the arithmetic, is what those kernels wait for.  Here a thread owns sixteen
// points, so one stage can be a radix-16 butterfly and N = 2048 = 16 x 16 x 8 needs TWO exchanges
// (1024 = 16 x 8 x 8, 512 = 8 x 8 x 8, 256 = 8 x 8 x 4: two; 128 = 16 x 8, 64 = 8 x 8: one).  The first stage
// runs from the registers the caller filled (thread tid holds elements tid + m N/16, m < 16, exactly what a
// coalesced strided load produces), the last stage leaves the result in registers, and the butterflies of the
// last stage are dealt out in PAIRS (j, N/R - j): the thread that holds bin k also holds bin N - k, which is what
// the unpacking of two real signals from one complex transform (and its inverse, the Hermitian packing) needs.
// So no pass over shared memory exists for loading, unpacking or packing.
//
// Same conventions as fft.cuh: forward X[k] = sum x[n] exp(-2 pi i k n / N), unnormalised both ways, twiddle
// table tw[m] = exp(-2 pi i m / N), shared buffers indexed through pad().
#pragma once
#include "fft.cuh"

namespace dgfft16 {

using namespace dgfft;

// stage radices per transform size; R3 == 0: a two-stage transform
template <int N> struct Plan;
template <> struct Plan<2048> { static constexpr int R1 = 16, R2 = 16, R3 = 8; };
template <> struct Plan<1024> { static constexpr int R1 = 16, R2 = 8, R3 = 8; };
template <> struct Plan<512> { static constexpr int R1 = 8, R2 = 8, R3 = 8; };
template <> struct Plan<256> { static constexpr int R1 = 8, R2 = 8, R3 = 4; };
template <> struct Plan<128> { static constexpr int R1 = 16, R2 = 8, R3 = 0; };
template <> struct Plan<64> { static constexpr int R1 = 8, R2 = 8, R3 = 0; };

template <int N> struct Geo {
  static constexpr int T = N / 16;                                          // threads per transform
  static constexpr int RL = Plan<N>::R3 ? Plan<N>::R3 : Plan<N>::R2;        // radix of the last stage (<= 8)
  static constexpr int NBL = N / RL;                                        // butterflies of the last stage
  static constexpr int PAIRS = 8 / RL;                                      // butterfly pairs per thread there
  static constexpr bool THREE = Plan<N>::R3 != 0;
};

// Where element i of a stage's output sits in the transform's shared-memory buffer.  l1: written by the first stage
// (read by the middle stage, or by the last one of a two-stage transform); l2: written by the middle stage, read by
// the last.  Classic: pad() for both, padded(N) elements per transform.
struct LayoutClassic {
  template <int N> __device__ static __forceinline__ int l1(int i) { return pad(i); }
  template <int N> __device__ static __forceinline__ int l2(int i) { return pad(i); }
  template <int N> __host__ __device__ static constexpr int size() { return padded(N); }
};
// Conflict-free for every exchange of the forward transform run IN PLACE (8-byte elements, half-warps of 16 lanes
// over 16 bank pairs; found by enumerating the access patterns of a warp for every size and stage):
//   * the last stage reads butterfly j and its partner NBL - j: an ascending and a DESCENDING run of 16 lanes.
//     With a pad every 16 elements the descending run from a multiple of 16 straddles a pad and two of its lanes
//     meet (1.5 x the wavefronts); the middle stage's output needs no padding at all for N >= 1024 (its scatter
//     has stride 16), so there l2 is the identity;
//   * for N = 512 / 256 (first radix 8) the middle stage's scatter puts lanes k and k + 8 sixty-four elements
//     apart: a shift of 8 elements per 64 separates them (2 x before);
//   * for N = 64 the first stage's scatter (stride 8, eight transforms per warp) wants a pad every 8 elements and
//     76 elements per transform (2 x before).
struct LayoutFree {
  template <int N> __device__ static __forceinline__ int l1(int i) { return N == 64 ? i + (i >> 3) : pad(i); }
  template <int N> __device__ static __forceinline__ int l2(int i) {
    return N >= 1024 ? i : (N == 512 || N == 256) ? i + 8 * (i >> 6) : l1<N>(i);
  }
  template <int N> __host__ __device__ static constexpr int size() { return N == 64 ? 76 : N == 512 ? 568 : N == 256 ? 280 : padded(N); }
};

// multiply by exp(-+ 2 pi i m / 16), m a compile-time constant in 0..9
template <int M, bool INV>
__device__ __forceinline__ float2 mul_w16(float2 a) {
  constexpr float C1 = 0.92387953251128674f, S1 = 0.38268343236508977f, H = 0.70710678118654752f;
  // forward: (c - i s)
  if (M == 0) return a;
  if (M == 4) return rot90<INV>(a);
  float c, s;
  if (M == 1) { c = C1; s = S1; }
  else if (M == 2) { c = H; s = H; }
  else if (M == 3) { c = S1; s = C1; }
  else if (M == 6) { c = -H; s = H; }
  else /* M == 9 */ { c = -C1; s = -S1; }
  if (INV) s = -s;
  // (a.x + i a.y)(c - i s) = (a.x c + a.y s) + i (a.y c - a.x s)
  return make_float2(fmaf(a.x, c, a.y * s), fmaf(a.y, c, -a.x * s));
}

// 16-point DFT in registers, natural order in and out (4 x 4 decomposition)
template <bool INV>
__device__ __forceinline__ void dft16(float2 *v) {
#pragma unroll
  for (int r = 0; r < 4; ++r) dft4<INV>(v[r], v[r + 4], v[r + 8], v[r + 12]);
  // v[r + 4 q] = Y[r][q]; twiddle W16^(r q)
  v[5] = mul_w16<1, INV>(v[5]);   v[9] = mul_w16<2, INV>(v[9]);   v[13] = mul_w16<3, INV>(v[13]);
  v[6] = mul_w16<2, INV>(v[6]);   v[10] = mul_w16<4, INV>(v[10]); v[14] = mul_w16<6, INV>(v[14]);
  v[7] = mul_w16<3, INV>(v[7]);   v[11] = mul_w16<6, INV>(v[11]); v[15] = mul_w16<9, INV>(v[15]);
#pragma unroll
  for (int q = 0; q < 4; ++q) dft4<INV>(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  // v[4 q + s] = X[q + 4 s]: transpose the 4 x 4 register tile
#pragma unroll
  for (int q = 0; q < 4; ++q)
#pragma unroll
    for (int s = q + 1; s < 4; ++s) {
      float2 t = v[4 * q + s];
      v[4 * q + s] = v[4 * s + q];
      v[4 * s + q] = t;
    }
}

template <int R, bool INV>
__device__ __forceinline__ void dftN(float2 *v) {
  if (R == 16) dft16<INV>(v);
  else dftR<R, INV>(v);
}

// v[t] *= w^t for t = 1 .. R-1, w = tw[m] (conjugated for the inverse): powers 1, 2, 4 (, 8) come from the table,
// the others are products of those
template <int R, bool INV>
__device__ __forceinline__ void twiddle(float2 *v, const float2 *__restrict__ tw, int m) {
  auto ld = [&](int idx) {
    float2 w = __ldg(&tw[idx]);
    if (INV) w.y = -w.y;
    return w;
  };
  if (R == 2) {
    v[1] = cmul(v[1], ld(m));
  } else if (R == 4) {
    const float2 w1 = ld(m), w2 = ld(2 * m);
    v[1] = cmul(v[1], w1); v[2] = cmul(v[2], w2); v[3] = cmul(v[3], cmul(w1, w2));
  } else if (R == 8) {
    const float2 w1 = ld(m), w2 = ld(2 * m), w4 = ld(4 * m);
    const float2 w3 = cmul(w1, w2), w5 = cmul(w1, w4), w6 = cmul(w2, w4), w7 = cmul(w3, w4);
    v[1] = cmul(v[1], w1); v[2] = cmul(v[2], w2); v[3] = cmul(v[3], w3); v[4] = cmul(v[4], w4);
    v[5] = cmul(v[5], w5); v[6] = cmul(v[6], w6); v[7] = cmul(v[7], w7);
  } else {
    const float2 w1 = ld(m), w2 = ld(2 * m), w4 = ld(4 * m), w8 = ld(8 * m);
    const float2 w3 = cmul(w1, w2), w5 = cmul(w1, w4), w6 = cmul(w2, w4), w7 = cmul(w3, w4);
    v[1] = cmul(v[1], w1); v[2] = cmul(v[2], w2); v[3] = cmul(v[3], w3); v[4] = cmul(v[4], w4);
    v[5] = cmul(v[5], w5); v[6] = cmul(v[6], w6); v[7] = cmul(v[7], w7); v[8] = cmul(v[8], w8);
    v[9] = cmul(v[9], cmul(w1, w8)); v[10] = cmul(v[10], cmul(w2, w8)); v[11] = cmul(v[11], cmul(w3, w8));
    v[12] = cmul(v[12], cmul(w4, w8)); v[13] = cmul(v[13], cmul(w5, w8)); v[14] = cmul(v[14], cmul(w6, w8));
    v[15] = cmul(v[15], cmul(w7, w8));
  }
}

// the threads that share one transform wait for each other
template <int N>
__device__ __forceinline__ void sync_transform() {
  if (N / 16 <= 32) __syncwarp();
  else __syncthreads();   // callers give every transform of N >= 1024 whole warps and run them in lockstep
}

// First stage, from registers: x[m] = element tid + m T.  Writes the stage output to `buf` (Stockham order).
template <int N, bool INV, class LAY = LayoutClassic>
__device__ __forceinline__ void stage_first(float2 (&x)[16], float2 *buf, int tid) {
  constexpr int R = Plan<N>::R1, PER = 16 / R, T = N / 16;
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    float2 v[R];
#pragma unroll
    for (int t = 0; t < R; ++t) v[t] = x[q + PER * t];      // in[j + t N/R], j = tid + q T
    dftN<R, INV>(v);
    const int j = tid + q * T;
#pragma unroll
    for (int t = 0; t < R; ++t) buf[LAY::template l1<N>(j * R + t)] = v[t];
  }
}

// Middle stage: shared -> shared, input stride Ns = R1.
template <int N, bool INV, class LAY = LayoutClassic>
__device__ __forceinline__ void stage_middle(const float2 *in, float2 *out, int tid, const float2 *__restrict__ tw) {
  constexpr int R = Plan<N>::R2, PER = 16 / R, T = N / 16, Ns = Plan<N>::R1;
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    const int j = tid + q * T, k = j & (Ns - 1);
    float2 v[R];
#pragma unroll
    for (int t = 0; t < R; ++t) v[t] = in[LAY::template l1<N>(j + t * (N / R))];
    twiddle<R, INV>(v, tw, k * (N / (Ns * R)));
    dftN<R, INV>(v);
    const int j0 = (j - k) * R + k;
#pragma unroll
    for (int t = 0; t < R; ++t) out[LAY::template l2<N>(j0 + t * Ns)] = v[t];
  }
}

// The middle stage IN PLACE: every thread first reads all sixteen of its inputs, the threads of the transform wait
// for each other, then the butterflies run from the registers and their outputs go back into the same buffer.  One
// more wait per transform, half the shared memory: the transforms of a block then leave room for more resident
// blocks.
template <int N, bool INV, class LAY = LayoutClassic>
__device__ __forceinline__ void stage_middle_inplace(float2 *buf, int tid, const float2 *__restrict__ tw) {
  constexpr int R = Plan<N>::R2, PER = 16 / R, T = N / 16, Ns = Plan<N>::R1;
  float2 v[PER][R];
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    const int j = tid + q * T;
#pragma unroll
    for (int t = 0; t < R; ++t) v[q][t] = buf[LAY::template l1<N>(j + t * (N / R))];
  }
  sync_transform<N>();
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    const int j = tid + q * T, k = j & (Ns - 1);
    twiddle<R, INV>(v[q], tw, k * (N / (Ns * R)));
    dftN<R, INV>(v[q]);
    const int j0 = (j - k) * R + k;
#pragma unroll
    for (int t = 0; t < R; ++t) buf[LAY::template l2<N>(j0 + t * Ns)] = v[q][t];
  }
}

// The two butterflies of pair p of the last stage that thread tid owns: (a, NBL - a), or (0, NBL / 2) for a == 0.
template <int N>
__device__ __forceinline__ void last_pair(int tid, int p, int &ja, int &jb) {
  const int a = tid + p * (N / 16);
  ja = a;
  jb = a == 0 ? Geo<N>::NBL / 2 : Geo<N>::NBL - a;
}

// Last stage: shared -> registers.  z[p][0][t] = bin ja + t NBL, z[p][1][t] = bin jb + t NBL.
// For a != 0 the partner of bin (ja, t) is bin (jb, RL - 1 - t).
template <int N, bool INV, class LAY = LayoutClassic>
__device__ __forceinline__ void stage_last(const float2 *in, float2 (&z)[Geo<N>::PAIRS][2][Geo<N>::RL], int tid,
                                           const float2 *__restrict__ tw) {
  constexpr int R = Geo<N>::RL, NBL = Geo<N>::NBL;
#pragma unroll
  for (int p = 0; p < Geo<N>::PAIRS; ++p) {
    int jj[2];
    last_pair<N>(tid, p, jj[0], jj[1]);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int j = jj[e];
#pragma unroll
      for (int t = 0; t < R; ++t)
        z[p][e][t] = in[Geo<N>::THREE ? LAY::template l2<N>(j + t * NBL) : LAY::template l1<N>(j + t * NBL)];
      twiddle<R, INV>(z[p][e], tw, j);     // Ns = NBL: k = j, table step 1
      dftN<R, INV>(z[p][e]);
    }
  }
}

// Whole forward or inverse transform: registers x[16] in (element tid + m N/16), registers z out (see stage_last).
// bufa / bufb: padded(N) float2 each (bufb unused by the two-stage sizes); nobody may still read them on entry.
// bufb == bufa selects the in-place middle stage (one buffer per transform).
// LAY::size<N>() elements per transform buffer.
template <int N, bool INV, class LAY = LayoutClassic>
__device__ __forceinline__ void fft16(float2 (&x)[16], float2 (&z)[Geo<N>::PAIRS][2][Geo<N>::RL], float2 *bufa,
                                      float2 *bufb, int tid, const float2 *__restrict__ tw) {
  stage_first<N, INV, LAY>(x, bufa, tid);
  sync_transform<N>();
  if (Geo<N>::THREE) {
    if (bufb == bufa) stage_middle_inplace<N, INV, LAY>(bufa, tid, tw);
    else stage_middle<N, INV, LAY>(bufa, bufb, tid, tw);
    sync_transform<N>();
    stage_last<N, INV, LAY>(bufb, z, tid, tw);
  } else {
    stage_last<N, INV, LAY>(bufa, z, tid, tw);
  }
}

// ---------------------------------------------------------------------------------------------------------
// The transposed network.  The DFT matrix is symmetric, so running the three stages in REVERSE order, each one
// transposed (butterfly first, then the twiddles; reads where the forward stage wrote, writes where it read),
// computes the same transform -- but takes its input in the bin layout the forward leaves in registers
// (y[p][e][t] = bin j_e + t NBL of last_pair) and returns element tid + m N/16 in x[m].  A spectrum that was
// built in the registers of a forward transform's result therefore goes back to the time domain, in the
// layout a coalesced store (or the overlap-add) wants, without any reordering pass.
// ---------------------------------------------------------------------------------------------------------
// v[t] *= w^t, after the butterfly (same table access as twiddle())
template <int N, bool INV, class LAY = LayoutClassic>
__device__ __forceinline__ void stage_last_T(float2 (&y)[Geo<N>::PAIRS][2][Geo<N>::RL], float2 *out, int tid,
                                             const float2 *__restrict__ tw) {
  constexpr int R = Geo<N>::RL, NBL = Geo<N>::NBL;
#pragma unroll
  for (int p = 0; p < Geo<N>::PAIRS; ++p) {
    int jj[2];
    last_pair<N>(tid, p, jj[0], jj[1]);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int j = jj[e];
      dftN<R, INV>(y[p][e]);
      twiddle<R, INV>(y[p][e], tw, j);
#pragma unroll
      for (int t = 0; t < R; ++t)
        out[Geo<N>::THREE ? LAY::template l2<N>(j + t * NBL) : LAY::template l1<N>(j + t * NBL)] = y[p][e][t];
    }
  }
}

template <int N, bool INV, class LAY = LayoutClassic>
__device__ __forceinline__ void stage_middle_T(const float2 *in, float2 *out, int tid, const float2 *__restrict__ tw) {
  constexpr int R = Plan<N>::R2, PER = 16 / R, T = N / 16, Ns = Plan<N>::R1;
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    const int j = tid + q * T, k = j & (Ns - 1);
    const int j0 = (j - k) * R + k;
    float2 v[R];
#pragma unroll
    for (int t = 0; t < R; ++t) v[t] = in[LAY::template l2<N>(j0 + t * Ns)];
    dftN<R, INV>(v);
    twiddle<R, INV>(v, tw, k * (N / (Ns * R)));
#pragma unroll
    for (int t = 0; t < R; ++t) out[LAY::template l1<N>(j + t * (N / R))] = v[t];
  }
}

template <int N, bool INV, class LAY = LayoutClassic>
__device__ __forceinline__ void stage_first_T(const float2 *buf, float2 (&x)[16], int tid) {
  constexpr int R = Plan<N>::R1, PER = 16 / R, T = N / 16;
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    const int j = tid + q * T;
    float2 v[R];
#pragma unroll
    for (int t = 0; t < R; ++t) v[t] = buf[LAY::template l1<N>(j * R + t)];
    dftN<R, INV>(v);
#pragma unroll
    for (int t = 0; t < R; ++t) x[q + PER * t] = v[t];
  }
}

// Transform of a spectrum held in the forward's register layout: y in (destroyed), x[m] = element tid + m N/16 out.
// The first write goes to the buffer the forward's last stage read, so a caller that has just finished a forward
// transform with the same buffers only has to make sure (sync_transform) that every thread is done reading it.
template <int N, bool INV, class LAY = LayoutClassic>
__device__ __forceinline__ void fft16_T(float2 (&y)[Geo<N>::PAIRS][2][Geo<N>::RL], float2 (&x)[16], float2 *bufa,
                                        float2 *bufb, int tid, const float2 *__restrict__ tw) {
  if (Geo<N>::THREE) {
    stage_last_T<N, INV, LAY>(y, bufb, tid, tw);
    sync_transform<N>();
    stage_middle_T<N, INV, LAY>(bufb, bufa, tid, tw);
    sync_transform<N>();
  } else {
    stage_last_T<N, INV, LAY>(y, bufa, tid, tw);
    sync_transform<N>();
  }
  stage_first_T<N, INV, LAY>(bufa, x, tid);
}

}  // namespace dgfft16
