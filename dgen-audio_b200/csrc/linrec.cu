// Linear recurrences over time as chunked parallel scans: one-pole history feedback, the tensor
// biquad bank forward, and the reverse-time (BPTT) pass that yields coefficient gradients.
//
// The reference runs these per sample through history cells (Sources/DGen/Emit+State.swift:150-224,
// Sources/DGen/HigherOps.swift:401-570): one thread per lane, a serial loop over frames, and for
// BPTT a stored forward tape plus a reverse loop (Sources/DGen/Blocks/Emission/BPTTEmission.swift:471-518).
// Here time is cut into chunks; every (lane, chunk) runs the recurrence from a zero state, the
// chunk-to-chunk carry is an affine map (a power of the 2x2 transition matrix) resolved by a short
// scan, and a second sweep produces the output (forward) or the gradient sums (backward; by
// linearity the sums are corrected for the carried adjoint state without re-reading the signals).
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------
// one-pole  y[n] = x[n] + a*y[n-1]
// ---------------------------------------------------------------------------------------------
constexpr int OP_THREADS = 256, OP_PER = 8, OP_CHUNK = OP_THREADS * OP_PER;

// inclusive scan over the block of v_t = sum_{s<=t} r^(t-s) * e_s   (r = a^OP_PER), via shuffles
__device__ __forceinline__ float block_decay_scan(float e, const float *rpow /* r^(2^i), i<8 */, float *warp_tot,
                                                  int tid) {
  float v = e;
#pragma unroll
  for (int i = 0; i < 5; ++i) {
    float o = __shfl_up_sync(0xffffffffu, v, 1 << i);
    if ((tid & 31) >= (1 << i)) v = fmaf(rpow[i], o, v);
  }
  if ((tid & 31) == 31) warp_tot[tid >> 5] = v;
  __syncthreads();
  if (tid < 32) {
    float w = tid < OP_THREADS / 32 ? warp_tot[tid] : 0.0f;
    // scan over warps with multiplier r^32 = rpow[5], r^64, r^128
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      float o = __shfl_up_sync(0xffffffffu, w, 1 << i);
      if (tid >= (1 << i)) w = fmaf(rpow[5 + i], o, w);
    }
    if (tid < OP_THREADS / 32) warp_tot[tid] = w;
  }
  __syncthreads();
  if (tid >= 32) {
    // add the carry of all previous warps, decayed by r^(lane+1)
    float carry = warp_tot[(tid >> 5) - 1];
    float d = rpow[8 + (tid & 31)];
    v = fmaf(d, carry, v);
  }
  return v;
}

// phase 0: chunk end values with zero carry-in; phase 1: final output using carry[chunk]
// REV: the same scan run backwards in time (frame n of the scan is memory index T-1-n): the adjoint recursion
// lam[n] = g[n] + a lam[n+1] of the filter's backward pass.
template <int PHASE, bool REV = false>
__global__ void __launch_bounds__(OP_THREADS)
onepole_kernel(const float *__restrict__ x, int T, int NC, float a, const float *__restrict__ carry_in,
               float *__restrict__ chunk_end, float *__restrict__ y) {
  __shared__ float rpow[8 + 32];
  __shared__ float warp_tot[OP_THREADS / 32];
  const int tid = threadIdx.x, c = blockIdx.x, b = blockIdx.y;
  if (tid == 0) {
    float r = 1.0f;
    for (int i = 0; i < OP_PER; ++i) r *= a;  // a^OP_PER
    float p = r;
    for (int i = 0; i < 8; ++i) { rpow[i] = p; p *= p; }
    float q = r;
    for (int i = 0; i < 32; ++i) { rpow[8 + i] = q; q *= r; }  // r^(i+1)
  }
  __syncthreads();
  const float *xb = x + (size_t)b * T;
  const int n0 = c * OP_CHUNK + tid * OP_PER;
  float loc[OP_PER];
  float prev = 0.0f;
  static_assert(OP_PER == 8, "the vector path moves a thread's run as two 128-bit words");
  // a thread's run of eight frames is 32 contiguous bytes: two 128-bit accesses when the voice row is aligned
  // memory index of the run's lowest address: n0 forwards, T - n0 - 8 backwards (the run is then read high to low)
  const int m0 = REV ? T - n0 - OP_PER : n0;
  const bool vec = n0 + OP_PER <= T && ((((uintptr_t)(xb + m0)) | (PHASE == 1 ? (uintptr_t)(y + (size_t)b * T + m0) : 0)) & 15) == 0;
  if (vec) {
    const float4 u = __ldg(reinterpret_cast<const float4 *>(xb + m0)), w = __ldg(reinterpret_cast<const float4 *>(xb + m0) + 1);
    if (REV) {
      loc[7] = u.x; loc[6] = u.y; loc[5] = u.z; loc[4] = u.w;
      loc[3] = w.x; loc[2] = w.y; loc[1] = w.z; loc[0] = w.w;
    } else {
      loc[0] = u.x; loc[1] = u.y; loc[2] = u.z; loc[3] = u.w;
      loc[4] = w.x; loc[5] = w.y; loc[6] = w.z; loc[7] = w.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < OP_PER; ++j) loc[j] = (n0 + j < T) ? xb[REV ? T - 1 - (n0 + j) : n0 + j] : 0.0f;
  }
#pragma unroll
  for (int j = 0; j < OP_PER; ++j) {
    prev = fmaf(a, prev, loc[j]);
    loc[j] = prev;
  }
  float incl = block_decay_scan(prev, rpow, warp_tot, tid);  // state at the end of this thread's run
  if (PHASE == 0) {
    if (tid == OP_THREADS - 1) chunk_end[(size_t)b * NC + c] = incl;
    return;
  }
  // state entering this thread's run = (incl - prev)/... simpler: exclusive value via shuffle
  float excl = __shfl_up_sync(0xffffffffu, incl, 1);
  __shared__ float last_of_warp[OP_THREADS / 32];
  if ((tid & 31) == 31) last_of_warp[tid >> 5] = incl;
  __syncthreads();
  if ((tid & 31) == 0) excl = tid == 0 ? 0.0f : last_of_warp[(tid >> 5) - 1];
  // carry from previous chunks decays by a^(tid*OP_PER) before reaching this thread
  float cin = carry_in[(size_t)b * NC + c];
  float dec = 1.0f;
  {
    // a^(tid*OP_PER) = r^tid from the binary powers
    int e = tid;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (e & (1 << i)) dec *= rpow[i];
  }
  float state = fmaf(dec, cin, excl);
  float *yb = y + (size_t)b * T;
  float ap = a;
#pragma unroll
  for (int j = 0; j < OP_PER; ++j) {
    loc[j] = fmaf(ap, state, loc[j]);
    ap *= a;
  }
  if (vec && REV) {
    __stcs(reinterpret_cast<float4 *>(yb + m0), make_float4(loc[7], loc[6], loc[5], loc[4]));
    __stcs(reinterpret_cast<float4 *>(yb + m0) + 1, make_float4(loc[3], loc[2], loc[1], loc[0]));
  } else if (vec) {
    __stcs(reinterpret_cast<float4 *>(yb + n0), make_float4(loc[0], loc[1], loc[2], loc[3]));
    __stcs(reinterpret_cast<float4 *>(yb + n0) + 1, make_float4(loc[4], loc[5], loc[6], loc[7]));
  } else {
#pragma unroll
    for (int j = 0; j < OP_PER; ++j)
      if (n0 + j < T) yb[REV ? T - 1 - (n0 + j) : n0 + j] = loc[j];
  }
}

// carry[c] = state entering chunk c; serial over chunks (few), one thread per voice
// y0_dev (optional): per-voice state entering the first chunk (the history cell before the call), else y0
__global__ void onepole_carry_kernel(const float *__restrict__ chunk_end, int B, int NC, float a, float y0,
                                     float *__restrict__ carry, const float *__restrict__ y0_dev = nullptr) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  float ac = 1.0f;
  for (int i = 0; i < OP_CHUNK; ++i) ac *= a;
  float s = y0_dev ? y0_dev[b] : y0;
  for (int c = 0; c < NC; ++c) {
    carry[(size_t)b * NC + c] = s;
    s = fmaf(ac, s, chunk_end[(size_t)b * NC + c]);
  }
}

// ---------------------------------------------------------------------------------------------
// biquad bank
// ---------------------------------------------------------------------------------------------
constexpr int BQ_CHUNK = 512;     // frames per (lane, chunk) thread
constexpr int BQ_THREADS = 128;   // lanes per block

// value with derivatives w.r.t. cutoff and q
struct Dual {
  float v, dc, dq;
};
__device__ __forceinline__ Dual dmul(Dual a, Dual b) { return {a.v * b.v, a.dc * b.v + a.v * b.dc, a.dq * b.v + a.v * b.dq}; }
__device__ __forceinline__ Dual dadd(Dual a, Dual b) { return {a.v + b.v, a.dc + b.dc, a.dq + b.dq}; }
__device__ __forceinline__ Dual dsub(Dual a, Dual b) { return {a.v - b.v, a.dc - b.dc, a.dq - b.dq}; }
__device__ __forceinline__ Dual ddiv(Dual a, Dual b) {
  float q = a.v / b.v;
  return {q, (a.dc - q * b.dc) / b.v, (a.dq - q * b.dq) / b.v};
}
__device__ __forceinline__ Dual dconst(float c) { return {c, 0.f, 0.f}; }
__device__ __forceinline__ Dual dabs(Dual a) { return a.v < 0.f ? Dual{-a.v, -a.dc, -a.dq} : a; }

__device__ __forceinline__ Dual dselect(float mode1, const Dual *opt, int n) {
  if (mode1 <= 0.f) return dconst(0.f);
  for (int i = 0; i < n; ++i)
    if (mode1 <= (float)(i + 1)) return opt[i];
  return dconst(0.f);
}

// Graph.biquad coefficient DAG (Sources/DGen/HigherOps.swift:444-555), all eight modes, node by node.
// coef layout per lane: b0 b1 b2 a1 a2, then d/dcutoff of the five, then d/dq of the five.
__global__ void biquad_coef_kernel(const float *__restrict__ cutoff, const float *__restrict__ q, int L, float gain,
                                   float mode, float *__restrict__ coef) {
  int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= L) return;
  Dual cut = {cutoff[l], 1.f, 0.f}, res = {q[l], 0.f, 1.f};
  float add4 = mode + 1.0f;
  Dual mult7 = dmul(dabs(cut), dconst(0.00014247585730565955f));
  Dual cos8 = {cosf(mult7.v), -sinf(mult7.v) * mult7.dc, -sinf(mult7.v) * mult7.dq};
  Dual mult9 = dmul(cos8, dconst(-1.f));
  Dual add10 = dadd(mult9, dconst(1.f));
  Dual div11 = ddiv(add10, dconst(2.f));
  Dual sub12 = dsub(mult9, dconst(1.f));
  Dual div13 = ddiv(sub12, dconst(-2.f));
  Dual sin14 = {sinf(mult7.v), cosf(mult7.v) * mult7.dc, cosf(mult7.v) * mult7.dq};
  Dual mult15 = dmul(sin14, dconst(0.5f));
  Dual abs17 = dabs(res);
  Dual div18 = ddiv(mult15, abs17);
  Dual mult19 = dmul(div18, dconst(-1.f));
  Dual mult20 = dmul(div18, abs17);
  Dual mult21 = dmul(mult20, dconst(-1.f));
  Dual add22 = dadd(div18, dconst(1.f));
  Dual recip24 = ddiv(dconst(1.f), add22);
  Dual mult26 = dmul(recip24, dconst(gain));
  Dual mult31 = dmul(mult9, dconst(2.f));
  Dual not_sub35 = dsub(dconst(1.f), div18);
  // shelf coefficients, modes 6 (high shelf) and 7 (low shelf): HigherOps.swift:468-528; A depends on the gain only
  const float Af = sqrtf(fabsf(gain));
  Dual A = dconst(Af);
  Dual cosW0Pos = dmul(mult9, dconst(-1.f));
  Dual alphaShelf = ddiv(sin14, dmul(dconst(2.0f), abs17));
  Dual Ap1 = dconst(Af + 1.0f), Am1 = dconst(Af - 1.0f);
  Dual Ap1_cos = dmul(Ap1, cosW0Pos), Am1_cos = dmul(Am1, cosW0Pos);
  Dual tsa = dmul(dconst(2.0f * sqrtf(Af)), alphaShelf);
  Dual hs_b0 = dmul(A, dadd(dadd(Ap1, Am1_cos), tsa));
  Dual hs_b1 = dmul(dconst(-2.0f), dmul(A, dadd(Am1, Ap1_cos)));
  Dual hs_b2 = dmul(A, dsub(dadd(Ap1, Am1_cos), tsa));
  Dual hs_a0 = dadd(dsub(Ap1, Am1_cos), tsa);
  Dual ls_b0 = dmul(A, dadd(dsub(Ap1, Am1_cos), tsa));
  Dual ls_b1 = dmul(dconst(2.0f), dmul(A, dsub(Am1, Ap1_cos)));
  Dual ls_b2 = dmul(A, dsub(dsub(Ap1, Am1_cos), tsa));
  Dual ls_a0 = dadd(dadd(Ap1, Am1_cos), tsa);
  Dual hs_a1n = ddiv(dmul(dconst(2.0f), dsub(Am1, Ap1_cos)), hs_a0), hs_a2n = ddiv(dsub(dsub(Ap1, Am1_cos), tsa), hs_a0);
  Dual ls_a1n = ddiv(dmul(dconst(-2.0f), dadd(Am1, Ap1_cos)), ls_a0), ls_a2n = ddiv(dsub(dadd(Ap1, Am1_cos), tsa), ls_a0);
  Dual o23[8] = {div11, div13, mult19, mult21, dconst(1.f), add22, ddiv(hs_b2, hs_a0), ddiv(ls_b2, ls_a0)};
  Dual o32[8] = {add10, sub12, dconst(0.f), dconst(0.f), mult31, mult31, ddiv(hs_b1, hs_a0), ddiv(ls_b1, ls_a0)};
  Dual o36[8] = {div11, div13, div18, mult20, dconst(1.f), not_sub35, ddiv(hs_b0, hs_a0), ddiv(ls_b0, ls_a0)};
  // modes 0-5 scale by gain / a0; the shelves carry the gain in A (isShelfMode = mode >= 6, :533-548)
  const bool shelf = mode >= 6.0f;
  Dual s23 = dselect(add4, o23, 8), s32 = dselect(add4, o32, 8), s36 = dselect(add4, o36, 8);
  Dual b2 = shelf ? s23 : dmul(s23, mult26);
  Dual b1 = shelf ? s32 : dmul(s32, mult26);
  Dual b0 = shelf ? s36 : dmul(s36, mult26);
  Dual a2 = shelf ? (mode >= 7.0f ? ls_a2n : hs_a2n) : dmul(not_sub35, recip24);
  Dual a1 = shelf ? (mode >= 7.0f ? ls_a1n : hs_a1n) : dmul(mult31, recip24);
  float *c = coef + (size_t)l * 15;
  c[0] = b0.v; c[1] = b1.v; c[2] = b2.v; c[3] = a1.v; c[4] = a2.v;
  c[5] = b0.dc; c[6] = b1.dc; c[7] = b2.dc; c[8] = a1.dc; c[9] = a2.dc;
  c[10] = b0.dq; c[11] = b1.dq; c[12] = b2.dq; c[13] = a1.dq; c[14] = a2.dq;
}

struct Coef {
  float b0, b1, b2, a1, a2;
};
__device__ __forceinline__ Coef load_coef(const float *coef, int l) {
  const float *c = coef + (size_t)l * 15;
  return {c[0], c[1], c[2], c[3], c[4]};
}

// y = ((b2*x2 + b1*x1) + b0*x0) - (a2*y2 + a1*y1), each operation rounded as in the reference graph
__device__ __forceinline__ float biquad_step(const Coef &c, float x0, float x1, float x2, float y1, float y2) {
  float add39 = __fadd_rn(__fadd_rn(__fmul_rn(x2, c.b2), __fmul_rn(x1, c.b1)), __fmul_rn(x0, c.b0));
  float add45 = __fadd_rn(__fmul_rn(y2, c.a2), __fmul_rn(y1, c.a1));
  return __fsub_rn(add39, add45);
}

// Per lane: the homogeneous transition over one chunk, M = [[m11 m12],[m21 m22]] with
// (y1,y2)_end = M (y1,y2)_start for zero input.  Poles close to the unit circle make the entries of
// M large with cancelling signs, so M and the chunk-to-chunk carry are kept in double precision.
__global__ void biquad_trans_kernel(const float *__restrict__ coef, int L, int len, double *__restrict__ trans) {
  int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= L) return;
  Coef c = load_coef(coef, l);
  const double a1 = c.a1, a2 = c.a2;
  double m[4];
  for (int col = 0; col < 2; ++col) {
    double y1 = col == 0 ? 1.0 : 0.0, y2 = col == 0 ? 0.0 : 1.0;
    for (int n = 0; n < len; ++n) {
      double v = -(a2 * y2 + a1 * y1);
      y2 = y1;
      y1 = v;
    }
    m[col] = y1;      // m11, m12
    m[2 + col] = y2;  // m21, m22
  }
  for (int i = 0; i < 4; ++i) trans[(size_t)l * 4 + i] = m[i];
}

// Forward sweep.  PHASE 0: end state of every (voice, lane, chunk) from a zero y-state.
//                 PHASE 1: rerun from the carried state and write y[b][n][l] (lanes fastest).
template <int PHASE>
__global__ void __launch_bounds__(BQ_THREADS)
biquad_fwd_kernel(const float *__restrict__ x, const float *__restrict__ coef, int B, int T, int L, int NC,
                  float *__restrict__ state /* [B][NC][L][2] */, float *__restrict__ y,
                  const float *__restrict__ st0 = nullptr /* [B][4][L]: history cells before the call */) {
  const int l = blockIdx.x * BQ_THREADS + threadIdx.x, c = blockIdx.y, b = blockIdx.z;
  __shared__ float xs[BQ_CHUNK + 2];
  const float *xb = x + (size_t)b * T;
  const int n0 = c * BQ_CHUNK, len = min(BQ_CHUNK, T - n0);
  for (int i = threadIdx.x; i < len + 2; i += BQ_THREADS) {
    int t = n0 - 2 + i;
    xs[i] = t >= 0 ? xb[t] : 0.0f;
  }
  __syncthreads();
  if (l >= L) return;
  const Coef cf = load_coef(coef, l);
  float *st = state + (((size_t)b * NC + c) * L + l) * 2;
  float y1 = 0.f, y2 = 0.f;
  if (PHASE == 1) {
    y1 = st[0];
    y2 = st[1];
  }
  float x2 = xs[0], x1 = xs[1];
  if (st0 && c == 0) {   // x[-1], x[-2] come from the history cells
    x1 = st0[((size_t)b * 4 + 2) * L + l];
    x2 = st0[((size_t)b * 4 + 3) * L + l];
  }
  float *yo = y + ((size_t)b * T + n0) * L + l;
#pragma unroll 4
  for (int n = 0; n < len; ++n) {
    float x0 = xs[n + 2];
    float v = biquad_step(cf, x0, x1, x2, y1, y2);
    if (PHASE == 1) yo[(size_t)n * L] = v;
    x2 = x1; x1 = x0; y2 = y1; y1 = v;
  }
  if (PHASE == 0) {
    st[0] = y1;
    st[1] = y2;
  }
}

// End state of a chunk as a LINEAR functional of its input.  Run from a zero y-state, the state (y[end], y[end-1])
// of lane l after a chunk is sum_m G[2l+s][m] * x[n0+m] plus two terms for the x-history x[n0-1], x[n0-2]:
//   hy[0] = 1, hy[k] = -a1 hy[k-1] - a2 hy[k-2]                  (response of the recursion to a unit drive)
//   h[k]  = b0 hy[k] + b1 hy[k-1] + b2 hy[k-2]                   (impulse response of the filter)
//   G[2l+0][m] = h[C-1-m], G[2l+1][m] = h[C-2-m]
//   history:  x[n0-1] -> (b1 hy[C-1] + b2 hy[C-2], b1 hy[C-2] + b2 hy[C-3]),  x[n0-2] -> (b2 hy[C-1], b2 hy[C-2])
// With that table the first pass of the forward -- the end state of EVERY (voice, chunk, lane) -- is one matrix
// product X[B*NC][C] * G^T[C][2L] on the tensor cores (its result lands directly in the [B][NC][L][2] state
// layout) instead of a second run of the serial recurrence.  The table is evaluated in double per call (the
// coefficients are inputs) and rounded once.
__global__ void biquad_endstate_table_kernel(const float *__restrict__ coef, int L, float *__restrict__ G,
                                             float *__restrict__ hist /* [L][4] */) {
  const int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= L) return;
  const Coef c = load_coef(coef, l);
  const double a1 = c.a1, a2 = c.a2, b0 = c.b0, b1 = c.b1, b2 = c.b2;
  float *g1 = G + (size_t)(2 * l) * BQ_CHUNK, *g2 = g1 + BQ_CHUNK;
  double hm1 = 0.0, hm2 = 0.0;   // hy[k-1], hy[k-2]
  double hprev = 0.0;            // h[k-1]
  double hyC1 = 0, hyC2 = 0, hyC3 = 0;
  for (int k = 0; k < BQ_CHUNK; ++k) {
    const double hy = k == 0 ? 1.0 : -(a2 * hm2 + a1 * hm1);
    const double h = b0 * hy + b1 * hm1 + b2 * hm2;
    // h[k] multiplies x[n0 + C-1-k] in y[end] and x[n0 + C-2-k] in y[end-1]
    g1[BQ_CHUNK - 1 - k] = (float)h;
    if (k >= 1) g2[BQ_CHUNK - 1 - k] = (float)hprev;   // h[k-1] at m = C-1-k  <=>  h[C-2-m]
    if (k == BQ_CHUNK - 1) {
      g2[BQ_CHUNK - 1] = 0.0f;                         // m = C-1: h[-1] = 0
      hyC1 = hy; hyC2 = hm1; hyC3 = hm2;
    }
    hprev = h;
    hm2 = hm1;
    hm1 = hy;
  }
  hist[l * 4 + 0] = (float)(b1 * hyC1 + b2 * hyC2);
  hist[l * 4 + 1] = (float)(b1 * hyC2 + b2 * hyC3);
  hist[l * 4 + 2] = (float)(b2 * hyC1);
  hist[l * 4 + 3] = (float)(b2 * hyC2);
}

// adds the x-history terms to the matrix-product states
__global__ void biquad_state_hist_kernel(const float *__restrict__ x, const float *__restrict__ hist, int B, int T, int L,
                                         int NC, float *__restrict__ state, const float *__restrict__ st0 = nullptr) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)B * NC * L) return;
  const int l = (int)(idx % L);
  const size_t bc = idx / L;
  const int c = (int)(bc % NC), b = (int)(bc / NC);
  if (c == 0 && !st0) return;   // no history before the first chunk
  const float *xb = x + (size_t)b * T + (size_t)c * BQ_CHUNK;
  const float x1 = c == 0 ? st0[((size_t)b * 4 + 2) * L + l] : xb[-1];
  const float x2 = c == 0 ? st0[((size_t)b * 4 + 3) * L + l] : xb[-2];
  float2 *st = reinterpret_cast<float2 *>(state) + idx;
  float2 v = *st;
  v.x += hist[l * 4 + 0] * x1 + hist[l * 4 + 2] * x2;
  v.y += hist[l * 4 + 1] * x1 + hist[l * 4 + 3] * x2;
  *st = v;
}

// The same sweep with FOUR lanes per thread (L a multiple of 4): four independent recurrences hide the
// latency of the dependent multiply-adds of one, and the output goes out as one 128-bit store per frame and
// thread (a warp writes 512 contiguous bytes).  Block = (L/4 lane quads, up to 4 chunks).
constexpr int BQ4_CHUNKS = 4;
template <int PHASE>
__global__ void __launch_bounds__(256)
biquad_fwd4_kernel(const float *__restrict__ x, const float *__restrict__ coef, int B, int T, int L, int NC,
                   float *__restrict__ state /* [B][NC][L][2] */, float *__restrict__ y,
                   const float *__restrict__ st0 = nullptr /* [B][4][L]: history cells before the call */) {
  __shared__ float xs[BQ4_CHUNKS][BQ_CHUNK + 2];
  const int lq = blockIdx.x * blockDim.x + threadIdx.x, cy = threadIdx.y;
  const int c = blockIdx.y * BQ4_CHUNKS + cy, b = blockIdx.z;
  const bool chunk_ok = c < NC;
  const float *xb = x + (size_t)b * T;
  const int n0 = c * BQ_CHUNK, len = chunk_ok ? min(BQ_CHUNK, T - n0) : 0;
  for (int i = threadIdx.x; i < len + 2; i += blockDim.x) {
    int t = n0 - 2 + i;
    xs[cy][i] = t >= 0 ? xb[t] : 0.0f;
  }
  __syncthreads();
  if (!chunk_ok || 4 * lq >= L) return;
  Coef cf[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) cf[k] = load_coef(coef, 4 * lq + k);
  float *st = state + (((size_t)b * NC + c) * L + 4 * lq) * 2;
  float y1[4] = {0.f, 0.f, 0.f, 0.f}, y2[4] = {0.f, 0.f, 0.f, 0.f};
  if (PHASE == 1) {
    const float4 s0 = *reinterpret_cast<const float4 *>(st), s1 = *reinterpret_cast<const float4 *>(st + 4);
    y1[0] = s0.x; y2[0] = s0.y; y1[1] = s0.z; y2[1] = s0.w;
    y1[2] = s1.x; y2[2] = s1.y; y1[3] = s1.z; y2[3] = s1.w;
  }
  float x2 = xs[cy][0], x1 = xs[cy][1];
  if (st0 && c == 0) {   // x[-1], x[-2] come from the history cells (one input feeds all lanes: the first lane's)
    x1 = st0[((size_t)b * 4 + 2) * L + 4 * lq];
    x2 = st0[((size_t)b * 4 + 3) * L + 4 * lq];
  }
  float *yo = y + ((size_t)b * T + n0) * L + 4 * lq;
#pragma unroll 2
  for (int n = 0; n < len; ++n) {
    const float x0 = xs[cy][n + 2];
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[k] = biquad_step(cf[k], x0, x1, x2, y1[k], y2[k]);
      y2[k] = y1[k];
      y1[k] = v[k];
    }
    if (PHASE == 1) __stcs(reinterpret_cast<float4 *>(yo + (size_t)n * L), make_float4(v[0], v[1], v[2], v[3]));
    x2 = x1;
    x1 = x0;
  }
  if (PHASE == 0) {
    *reinterpret_cast<float4 *>(st) = make_float4(y1[0], y2[0], y1[1], y2[1]);
    *reinterpret_cast<float4 *>(st + 4) = make_float4(y1[2], y2[2], y1[3], y2[3]);
  }
}

// state[c] <- state entering chunk c (exclusive scan of the affine maps), thread per (voice, lane)
__global__ void biquad_carry_kernel(const double *__restrict__ trans, int B, int L, int NC,
                                    float *__restrict__ state, const float *__restrict__ st0 = nullptr) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * L) return;
  int b = idx / L, l = idx - b * L;
  const double m11 = trans[(size_t)l * 4], m12 = trans[(size_t)l * 4 + 1], m21 = trans[(size_t)l * 4 + 2],
               m22 = trans[(size_t)l * 4 + 3];
  // y[-1], y[-2]: the history cells before the call, else rest
  double s1 = st0 ? (double)st0[((size_t)b * 4 + 0) * L + l] : 0.0, s2 = st0 ? (double)st0[((size_t)b * 4 + 1) * L + l] : 0.0;
  for (int c = 0; c < NC; ++c) {
    float *st = state + (((size_t)b * NC + c) * L + l) * 2;
    double e1 = st[0], e2 = st[1];
    st[0] = (float)s1;
    st[1] = (float)s2;
    // every chunk but possibly the last has full length; the state after the last chunk is unused
    double n1 = m11 * s1 + m12 * s2 + e1, n2 = m21 * s1 + m22 * s2 + e2;
    s1 = n1;
    s2 = n2;
  }
}

// Backward sweep for loss = scale * sum (y - t)^2.  Adjoint recurrence (transposed filter, reverse time):
//   lam[n] = g[n] - a1*lam[n+1] - a2*lam[n+2],  g = 2*scale*(y - t)
//   dL/db0 = sum lam[n] x[n], dL/db1 = sum lam[n] x[n-1], dL/db2 = sum lam[n] x[n-2],
//   dL/da1 = -sum lam[n] y[n-1], dL/da2 = -sum lam[n] y[n-2].
// One sweep per (voice, lane, chunk) from a zero terminal adjoint accumulates the five sums for the
// local adjoint AND for the two homogeneous adjoint responses h1, h2 (terminal state (1,0) and (0,1));
// the carry kernel then supplies the true terminal state s of each chunk and the total is
// S_loc + s1*S_h1 + s2*S_h2.  Record per (voice, chunk, lane): 15 sums + local start adjoint (2) + sq error.
constexpr int BW_REC = 18;

// UP = false: g = gscale * (y - tgt) (the MSE loss, squared error summed on the way);  UP = true: `tgt` IS the
// upstream gradient dL/dy [B][T][L] of an arbitrary loss.
template <bool UP>
__global__ void __launch_bounds__(BQ_THREADS)
biquad_bwd_kernel(const float *__restrict__ x, const float *__restrict__ coef, const float *__restrict__ y,
                  const float *__restrict__ tgt, int B, int T, int L, int NC, float gscale,
                  float *__restrict__ rec /* [B][NC][BW_REC][L] */) {
  const int l = blockIdx.x * BQ_THREADS + threadIdx.x, c = blockIdx.y, b = blockIdx.z;
  __shared__ float xs[BQ_CHUNK + 2];
  const float *xb = x + (size_t)b * T;
  const int n0 = c * BQ_CHUNK, len = min(BQ_CHUNK, T - n0);
  for (int i = threadIdx.x; i < len + 2; i += BQ_THREADS) {
    int t = n0 - 2 + i;
    xs[i] = t >= 0 ? xb[t] : 0.0f;
  }
  __syncthreads();
  if (l >= L) return;
  const Coef cf = load_coef(coef, l);
  const float *yb = y + (size_t)b * T * L + l, *tb = tgt + (size_t)b * T * L + l;
  float la1 = 0.f, la2 = 0.f;            // lam[n+1], lam[n+2] (local)
  float h1a = 1.f, h1b = 0.f;            // homogeneous response to terminal (lam[n_end+1], lam[n_end+2]) = (1,0)
  float h2a = 0.f, h2b = 1.f;            // ... = (0,1)
  float S[15];
#pragma unroll
  for (int i = 0; i < 15; ++i) S[i] = 0.f;
  float sq = 0.f;
  // y[n-1], y[n-2] sliding from the top: prefetch y at n, n-1, n-2
  int nt = n0 + len - 1;
  float yc = yb[(size_t)nt * L];
  float ym1 = nt - 1 >= 0 ? yb[(size_t)(nt - 1) * L] : 0.f;
  auto body = [&](int n, float ym2, float tv) {
    float g;
    if (UP) {
      g = tv;
    } else {
      float d = yc - tv;
      sq = fmaf(d, d, sq);
      g = gscale * d;
    }
    float lam = g - (cf.a1 * la1 + cf.a2 * la2);
    float h1 = -(cf.a1 * h1a + cf.a2 * h1b);
    float h2 = -(cf.a1 * h2a + cf.a2 * h2b);
    float x0 = xs[n + 2], x1 = xs[n + 1], x2 = xs[n];
    S[0] = fmaf(lam, x0, S[0]); S[1] = fmaf(lam, x1, S[1]); S[2] = fmaf(lam, x2, S[2]);
    S[3] = fmaf(lam, ym1, S[3]); S[4] = fmaf(lam, ym2, S[4]);
    S[5] = fmaf(h1, x0, S[5]); S[6] = fmaf(h1, x1, S[6]); S[7] = fmaf(h1, x2, S[7]);
    S[8] = fmaf(h1, ym1, S[8]); S[9] = fmaf(h1, ym2, S[9]);
    S[10] = fmaf(h2, x0, S[10]); S[11] = fmaf(h2, x1, S[11]); S[12] = fmaf(h2, x2, S[12]);
    S[13] = fmaf(h2, ym1, S[13]); S[14] = fmaf(h2, ym2, S[14]);
    la2 = la1; la1 = lam;
    h1b = h1a; h1a = h1;
    h2b = h2a; h2a = h2;
    yc = ym1; ym1 = ym2;
  };
  if (len == BQ_CHUNK && n0 >= 2) {
    // interior chunk: every load is in range, so a group of sixteen frames issues its 32 loads before the
    // dependent recurrence steps (the sweep is bound by loads in flight, not by arithmetic)
    constexpr int G = 16;
    for (int nb = BQ_CHUNK - G; nb >= 0; nb -= G) {
      float yv[G], tv[G];
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const int t = n0 + nb + j;
        yv[j] = __ldcs(yb + (size_t)(t - 2) * L);
        tv[j] = __ldcs(tb + (size_t)t * L);
      }
#pragma unroll
      for (int j = G - 1; j >= 0; --j) body(nb + j, yv[j], tv[j]);
    }
  } else {
    for (int n = len - 1; n >= 0; --n) {
      int t = n0 + n;
      float ym2 = t - 2 >= 0 ? yb[(size_t)(t - 2) * L] : 0.f;
      body(n, ym2, tb[(size_t)t * L]);
    }
  }
  float *r = rec + ((size_t)b * NC + c) * BW_REC * L + l;
#pragma unroll
  for (int i = 0; i < 15; ++i) r[(size_t)i * L] = S[i];
  r[(size_t)15 * L] = la1;  // local adjoint at the first frame of the chunk: lam[n0]
  r[(size_t)16 * L] = la2;  // lam[n0+1]
  r[(size_t)17 * L] = sq;
}

// Reverse carry over chunks, thread per (voice, lane): resolves the terminal adjoint of every chunk,
// combines the sums, and writes per (voice, lane) the five coefficient-gradient sums and the squared error.
__global__ void biquad_bwd_carry_kernel(const float *__restrict__ rec, const float *__restrict__ coef, int B, int L,
                                        int NC, int T, double *__restrict__ acc /* [B][L][6] */,
                                        float2 *__restrict__ term /* [B][NC][L] or null */) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * L) return;
  int b = idx / L, l = idx - b * L;
  const Coef cf = load_coef(coef, l);
  // adjoint transition over a full chunk: (lam[n0], lam[n0+1]) = A (s1, s2) + local, with A from the
  // homogeneous responses; recompute A by running the recurrence (cheap, per thread)
  const double da1 = cf.a1, da2 = cf.a2;
  auto homog = [&](int len, double &a11, double &a12, double &a21, double &a22) {
    double p1 = 1.0, p2 = 0.0, q1 = 0.0, q2 = 1.0;
    for (int n = 0; n < len; ++n) {
      double v = -(da1 * p1 + da2 * p2);
      p2 = p1; p1 = v;
      double w = -(da1 * q1 + da2 * q2);
      q2 = q1; q1 = w;
    }
    a11 = p1; a21 = p2; a12 = q1; a22 = q2;
  };
  double f11, f12, f21, f22;
  homog(BQ_CHUNK, f11, f12, f21, f22);
  double G[5] = {0, 0, 0, 0, 0}, sq = 0;
  double s1 = 0.0, s2 = 0.0;  // terminal adjoint (lam[n_end+1], lam[n_end+2]) of the current chunk
  for (int c = NC - 1; c >= 0; --c) {
    const float *r = rec + ((size_t)b * NC + c) * BW_REC * L + l;
    if (term) term[((size_t)b * NC + c) * L + l] = make_float2((float)s1, (float)s2);
    for (int i = 0; i < 5; ++i)
      G[i] += (double)r[(size_t)i * L] + s1 * (double)r[(size_t)(5 + i) * L] + s2 * (double)r[(size_t)(10 + i) * L];
    sq += (double)r[(size_t)17 * L];
    int len = min(BQ_CHUNK, T - c * BQ_CHUNK);
    double a11 = f11, a12 = f12, a21 = f21, a22 = f22;
    if (len != BQ_CHUNK) homog(len, a11, a12, a21, a22);
    double n1 = a11 * s1 + a12 * s2 + (double)r[(size_t)15 * L];
    double n2 = a21 * s1 + a22 * s2 + (double)r[(size_t)16 * L];
    s1 = n1;
    s2 = n2;
  }
  double *o = acc + ((size_t)b * L + l) * 6;
  o[0] = G[0]; o[1] = G[1]; o[2] = G[2]; o[3] = -G[3]; o[4] = -G[4]; o[5] = sq;
}

// Gradient with respect to the INPUT x[b][n] (shared by the lanes): sum over lanes of
//   b0 lam[n] + b1 lam[n+1] + b2 lam[n+2]
// A second reverse sweep per (voice, lane, chunk), now from the chunk's TRUE terminal adjoint (resolved by the carry
// kernel), recomputes lam; the sum over the block's 128 lanes goes through a shared-memory tile of 32 frames, the
// sum over lane blocks through per-block partial rows that a last kernel adds in a fixed order.
constexpr int GX_FRAMES = 32;

template <bool UP>
__global__ void __launch_bounds__(BQ_THREADS)
biquad_gx_kernel(const float *__restrict__ coef, const float *__restrict__ y, const float *__restrict__ tgt,
                 const float2 *__restrict__ term, int B, int T, int L, int NC, float gscale,
                 float *__restrict__ part /* [gridDim.x][B][T] */) {
  __shared__ float red[GX_FRAMES][BQ_THREADS + 1];
  const int tid = threadIdx.x, l = blockIdx.x * BQ_THREADS + tid, c = blockIdx.y, b = blockIdx.z;
  const int n0 = c * BQ_CHUNK, len = min(BQ_CHUNK, T - n0);
  const bool live = l < L;
  Coef cf = {};
  float la1 = 0.f, la2 = 0.f;
  if (live) {
    cf = load_coef(coef, l);
    const float2 s = term[((size_t)b * NC + c) * L + l];
    la1 = s.x;
    la2 = s.y;
  }
  const float *yb = y + (size_t)b * T * L + l, *tb = tgt + (size_t)b * T * L + l;
  float *pb = part + ((size_t)blockIdx.x * B + b) * T;
  // groups of 32 frames from the end of the chunk; the last group (lowest frames) may be shorter
  for (int hi = len; hi > 0; hi -= GX_FRAMES) {
    const int lo = max(hi - GX_FRAMES, 0), cnt = hi - lo;
    float gv[GX_FRAMES];
    if (live) {
#pragma unroll
      for (int j = 0; j < GX_FRAMES; ++j) {
        const int t = n0 + lo + j;
        if (j < cnt) gv[j] = UP ? __ldcs(tb + (size_t)t * L) : gscale * (__ldcs(yb + (size_t)t * L) - __ldcs(tb + (size_t)t * L));
        else gv[j] = 0.f;
      }
    }
#pragma unroll
    for (int j = GX_FRAMES - 1; j >= 0; --j) {
      float contrib = 0.f;
      if (live && j < cnt) {
        const float lam = gv[j] - (cf.a1 * la1 + cf.a2 * la2);
        contrib = fmaf(cf.b0, lam, fmaf(cf.b1, la1, cf.b2 * la2));
        la2 = la1;
        la1 = lam;
      }
      red[j][tid] = contrib;
    }
    __syncthreads();
    // thread -> (frame j = tid / 4, quarter of the lanes): 32 adds, then the four quarters by shuffles
    {
      const int j = tid >> 2, seg = tid & 3;
      float sum = 0.f;
#pragma unroll 8
      for (int k = 0; k < BQ_THREADS / 4; ++k) sum += red[j][seg * (BQ_THREADS / 4) + ((k + tid) & (BQ_THREADS / 4 - 1))];
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (seg == 0 && j < cnt) pb[n0 + lo + j] = sum;
    }
    __syncthreads();
  }
}

__global__ void sum_partial_rows_kernel(const float *__restrict__ part, int nparts, size_t n, float *__restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += part[(size_t)p * n + i];
  out[i] = s;
}

// Sum over voices (fixed order), chain rule to cutoff and q, total loss.
__global__ void biquad_bwd_final_kernel(const double *__restrict__ acc, const float *__restrict__ coef, int B, int L,
                                        float loss_scale, float *__restrict__ gcut, float *__restrict__ gq,
                                        double *__restrict__ lane_loss) {
  int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= L) return;
  double G[5] = {0, 0, 0, 0, 0}, sq = 0;
  for (int b = 0; b < B; ++b) {
    const double *a = acc + ((size_t)b * L + l) * 6;
    for (int i = 0; i < 5; ++i) G[i] += a[i];
    sq += a[5];
  }
  const float *c = coef + (size_t)l * 15;
  double dc = 0, dq = 0;
  for (int i = 0; i < 5; ++i) {
    dc += G[i] * (double)c[5 + i];
    dq += G[i] * (double)c[10 + i];
  }
  gcut[l] = (float)dc;
  gq[l] = (float)dq;
  lane_loss[l] = sq * (double)loss_scale;
}

__global__ void sum_doubles_kernel(const double *__restrict__ v, int n, double *__restrict__ out) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  double t = 0;
  for (int i = 0; i < n; ++i) t += v[i];
  out[0] = t;
}

}  // namespace

DGC_EXPORT int32_t dgc_onepole_fwd(dgc_ctx *ctx, const float *x_dev, int32_t B, int32_t T, float a, float *y_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, x_dev && y_dev, "null pointer");
  DGC_REQUIRE(ctx, B > 0 && T > 0, "size out of range");
  const int NC = dgc_div_up(T, OP_CHUNK);
  float *scr = dgc_ctx_scratch(ctx, 2ull * B * NC + 8);
  if (!scr) return DGC_ERR_OOM;
  float *chunk_end = scr, *carry = scr + (size_t)B * NC;
  onepole_kernel<0><<<dim3(NC, B), OP_THREADS, 0, ctx->stream>>>(x_dev, T, NC, a, nullptr, chunk_end, nullptr);
  DGC_LAUNCHED(ctx, "onepole_pass0");
  onepole_carry_kernel<<<dgc_div_up(B, 64), 64, 0, ctx->stream>>>(chunk_end, B, NC, a, 0.0f, carry);
  DGC_LAUNCHED(ctx, "onepole_carry");
  onepole_kernel<1><<<dim3(NC, B), OP_THREADS, 0, ctx->stream>>>(x_dev, T, NC, a, carry, nullptr, y_dev);
  DGC_LAUNCHED(ctx, "onepole_pass1");
  return DGC_OK;
}

__global__ void onepole_final_state_kernel(const float *__restrict__ y, int B, int T, float *__restrict__ state) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) state[b] = y[(size_t)b * T + T - 1];
}

DGC_EXPORT int32_t dgc_onepole_fwd_state(dgc_ctx *ctx, const float *x_dev, int32_t B, int32_t T, float a,
                                         float *state_dev, float *y_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  if (!state_dev) return dgc_onepole_fwd(ctx, x_dev, B, T, a, y_dev);
  DGC_REQUIRE(ctx, x_dev && y_dev, "null pointer");
  DGC_REQUIRE(ctx, B > 0 && T > 0, "size out of range");
  const int NC = dgc_div_up(T, OP_CHUNK);
  float *scr = dgc_ctx_scratch(ctx, 2ull * B * NC + 8);
  if (!scr) return DGC_ERR_OOM;
  float *chunk_end = scr, *carry = scr + (size_t)B * NC;
  onepole_kernel<0><<<dim3(NC, B), OP_THREADS, 0, ctx->stream>>>(x_dev, T, NC, a, nullptr, chunk_end, nullptr);
  DGC_LAUNCHED(ctx, "onepole_pass0");
  onepole_carry_kernel<<<dgc_div_up(B, 64), 64, 0, ctx->stream>>>(chunk_end, B, NC, a, 0.0f, carry, state_dev);
  DGC_LAUNCHED(ctx, "onepole_carry");
  onepole_kernel<1><<<dim3(NC, B), OP_THREADS, 0, ctx->stream>>>(x_dev, T, NC, a, carry, nullptr, y_dev);
  DGC_LAUNCHED(ctx, "onepole_pass1");
  onepole_final_state_kernel<<<dgc_div_up(B, 128), 128, 0, ctx->stream>>>(y_dev, B, T, state_dev);
  DGC_LAUNCHED(ctx, "onepole_final_state");
  return DGC_OK;
}

static int32_t biquad_validate(dgc_ctx *ctx, const dgc_biquad_params *p) {
  DGC_REQUIRE(ctx, p->B > 0 && p->T > 0 && p->L > 0, "size out of range");
  DGC_REQUIRE(ctx, p->B <= 65535, "B must be <= 65535");
  DGC_REQUIRE(ctx, p->mode >= 0.0f && p->mode <= 7.0f, "mode must be in 0..7");
  return DGC_OK;
}

DGC_EXPORT uint64_t dgc_biquad_scratch_floats(const dgc_biquad_params *p, int32_t backward) {
  if (!p || p->B <= 0 || p->T <= 0 || p->L <= 0) return 0;
  uint64_t NC = (uint64_t)(p->T + BQ_CHUNK - 1) / BQ_CHUNK;
  uint64_t coef = (((uint64_t)p->L * 16 + (uint64_t)p->L * 8) + 3) & ~3ull;
  // forward: chunk states, then the end-state response table [2L][BQ_CHUNK] and its 4L history terms
  if (!backward) return coef + (((uint64_t)p->B * NC * p->L * 2 + 3) & ~3ull) + (uint64_t)p->L * (2 * BQ_CHUNK + 4) + 16;
  uint64_t rec = (uint64_t)p->B * NC * BW_REC * p->L;
  uint64_t base = coef + ((rec + 3) & ~3ull) + 2 * ((uint64_t)p->B * p->L * 6 + p->L) + 16;
  if (backward == 1) return base;
  // backward == 2 (dgc_biquad_bwd with the input gradient): terminal adjoints [B][NC][L] float2, partial rows
  uint64_t blocks = ((uint64_t)p->L + BQ_THREADS - 1) / BQ_THREADS;
  return base + 2 * (uint64_t)p->B * NC * p->L + blocks * (uint64_t)p->B * p->T + 16;
}

// history cells after the call: y[T-1], y[T-2], x[T-1], x[T-2] per (voice, lane); frames before the call come
// from the cells as they were
__global__ void biquad_final_state_kernel(const float *__restrict__ x, const float *__restrict__ y, int B, int T, int L,
                                          float *__restrict__ st) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * L) return;
  const int b = idx / L, l = idx - b * L;
  float *s = st + (size_t)b * 4 * L + l;
  const float *yb = y + (size_t)b * T * L + l, *xb = x + (size_t)b * T;
  const float oy1 = s[0], ox1 = s[2 * L];
  s[0] = yb[(size_t)(T - 1) * L];
  s[L] = T >= 2 ? yb[(size_t)(T - 2) * L] : oy1;
  s[2 * L] = xb[T - 1];
  s[3 * L] = T >= 2 ? xb[T - 2] : ox1;
}

static int32_t biquad_fwd_impl(dgc_ctx *ctx, const dgc_biquad_params *p, const float *x_dev, const float *cutoff_dev,
                               const float *q_dev, float *scratch_dev, float *st0, float *y_dev);

DGC_EXPORT int32_t dgc_biquad_fwd(dgc_ctx *ctx, const dgc_biquad_params *p, const float *x_dev,
                                  const float *cutoff_dev, const float *q_dev, float *scratch_dev, float *y_dev) {
  return biquad_fwd_impl(ctx, p, x_dev, cutoff_dev, q_dev, scratch_dev, nullptr, y_dev);
}

DGC_EXPORT int32_t dgc_biquad_fwd_state(dgc_ctx *ctx, const dgc_biquad_params *p, const float *x_dev,
                                        const float *cutoff_dev, const float *q_dev, float *scratch_dev,
                                        float *state_dev, float *y_dev) {
  return biquad_fwd_impl(ctx, p, x_dev, cutoff_dev, q_dev, scratch_dev, state_dev, y_dev);
}

static int32_t biquad_fwd_impl(dgc_ctx *ctx, const dgc_biquad_params *p, const float *x_dev, const float *cutoff_dev,
                               const float *q_dev, float *scratch_dev, float *st0, float *y_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, p && x_dev && cutoff_dev && q_dev && y_dev, "null pointer");
  int32_t rc = biquad_validate(ctx, p);
  if (rc != DGC_OK) return rc;
  const int B = p->B, T = p->T, L = p->L, NC = dgc_div_up(T, BQ_CHUNK);
  DGC_REQUIRE(ctx, NC <= 65535, "T too large");
  float *scr = scratch_dev ? scratch_dev : dgc_ctx_scratch(ctx, dgc_biquad_scratch_floats(p, 0));
  if (!scr) return DGC_ERR_OOM;
  DGC_REQUIRE(ctx, (((uintptr_t)scr) & 15) == 0, "scratch must be 16-byte aligned");
  float *coef = scr;
  double *trans = reinterpret_cast<double *>(scr + (size_t)L * 16);
  float *state = scr + ((((size_t)L * 24) + 3) & ~(size_t)3);
  biquad_coef_kernel<<<dgc_div_up(L, 128), 128, 0, ctx->stream>>>(cutoff_dev, q_dev, L, p->gain, p->mode, coef);
  DGC_LAUNCHED(ctx, "biquad_coef");
  biquad_trans_kernel<<<dgc_div_up(L, 128), 128, 0, ctx->stream>>>(coef, L, BQ_CHUNK, trans);
  DGC_LAUNCHED(ctx, "biquad_trans");
  // four lanes per thread when the lane count and the output alignment allow 128-bit accesses
  const bool quad = (L & 3) == 0 && L >= 16 && ((((uintptr_t)y_dev) | ((uintptr_t)state)) & 15) == 0;
  const int qx = quad ? (L / 4 >= 64 ? 64 : L / 4) : 0;
  dim3 grid(dgc_div_up(L, BQ_THREADS), NC, B);
  dim3 grid4(quad ? dgc_div_up(L / 4, qx) : 1, dgc_div_up(NC, BQ4_CHUNKS), B), block4(quad ? qx : 1, BQ4_CHUNKS);
  // first pass: chunk end states from a zero y-state -- as one tensor-core product when the chunks tile T exactly
  // and the problem is large enough for that path, else by running the recurrence
  const bool by_matmul = (T % BQ_CHUNK) == 0 && (double)B * NC * L >= (double)(1 << 16) && (((uintptr_t)x_dev) & 15) == 0;
  if (by_matmul) {
    float *G = state + ((((size_t)B * NC * L * 2) + 3) & ~(size_t)3), *hist = G + (size_t)L * 2 * BQ_CHUNK;
    biquad_endstate_table_kernel<<<dgc_div_up(L, 64), 64, 0, ctx->stream>>>(coef, L, G, hist);
    DGC_LAUNCHED(ctx, "biquad_endstate_table");
    rc = dgc_gemm_nt(ctx, x_dev, G, B * NC, 2 * L, BQ_CHUNK, state);
    if (rc != DGC_OK) return rc;
    biquad_state_hist_kernel<<<dgc_div_up((int64_t)B * NC * L, 256), 256, 0, ctx->stream>>>(x_dev, hist, B, T, L, NC, state, st0);
  } else if (quad) biquad_fwd4_kernel<0><<<grid4, block4, 0, ctx->stream>>>(x_dev, coef, B, T, L, NC, state, nullptr, st0);
  else biquad_fwd_kernel<0><<<grid, BQ_THREADS, 0, ctx->stream>>>(x_dev, coef, B, T, L, NC, state, nullptr, st0);
  DGC_LAUNCHED(ctx, "biquad_fwd_state");
  biquad_carry_kernel<<<dgc_div_up(B * L, 128), 128, 0, ctx->stream>>>(trans, B, L, NC, state, st0);
  DGC_LAUNCHED(ctx, "biquad_carry");
  if (quad) biquad_fwd4_kernel<1><<<grid4, block4, 0, ctx->stream>>>(x_dev, coef, B, T, L, NC, state, y_dev, st0);
  else biquad_fwd_kernel<1><<<grid, BQ_THREADS, 0, ctx->stream>>>(x_dev, coef, B, T, L, NC, state, y_dev, st0);
  DGC_LAUNCHED(ctx, "biquad_fwd_out");
  if (st0) {
    biquad_final_state_kernel<<<dgc_div_up(B * L, 128), 128, 0, ctx->stream>>>(x_dev, y_dev, B, T, L, st0);
    DGC_LAUNCHED(ctx, "biquad_final_state");
  }
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_biquad_mse_bwd(dgc_ctx *ctx, const dgc_biquad_params *p, const float *x_dev,
                                      const float *cutoff_dev, const float *q_dev, const float *y_dev,
                                      const float *target_dev, float loss_scale, float *scratch_dev,
                                      float *grad_cutoff_dev, float *grad_q_dev, double *loss_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, p && x_dev && cutoff_dev && q_dev && y_dev && target_dev && grad_cutoff_dev && grad_q_dev &&
                       loss_dev, "null pointer");
  int32_t rc = biquad_validate(ctx, p);
  if (rc != DGC_OK) return rc;
  const int B = p->B, T = p->T, L = p->L, NC = dgc_div_up(T, BQ_CHUNK);
  DGC_REQUIRE(ctx, NC <= 65535, "T too large");
  float *scr = scratch_dev ? scratch_dev : dgc_ctx_scratch(ctx, dgc_biquad_scratch_floats(p, 1));
  if (!scr) return DGC_ERR_OOM;
  DGC_REQUIRE(ctx, (((uintptr_t)scr) & 15) == 0, "scratch must be 16-byte aligned");
  float *coef = scr;
  float *rec = scr + ((((size_t)L * 24) + 3) & ~(size_t)3);
  size_t rec_n = ((size_t)B * NC * BW_REC * L + 3) & ~(size_t)3;
  double *acc = reinterpret_cast<double *>(rec + rec_n);
  double *lane_loss = acc + (size_t)B * L * 6;
  biquad_coef_kernel<<<dgc_div_up(L, 128), 128, 0, ctx->stream>>>(cutoff_dev, q_dev, L, p->gain, p->mode, coef);
  DGC_LAUNCHED(ctx, "biquad_coef");
  dim3 grid(dgc_div_up(L, BQ_THREADS), NC, B);
  biquad_bwd_kernel<false><<<grid, BQ_THREADS, 0, ctx->stream>>>(x_dev, coef, y_dev, target_dev, B, T, L, NC,
                                                                 2.0f * loss_scale, rec);
  DGC_LAUNCHED(ctx, "biquad_bwd");
  biquad_bwd_carry_kernel<<<dgc_div_up(B * L, 128), 128, 0, ctx->stream>>>(rec, coef, B, L, NC, T, acc, nullptr);
  DGC_LAUNCHED(ctx, "biquad_bwd_carry");
  biquad_bwd_final_kernel<<<dgc_div_up(L, 128), 128, 0, ctx->stream>>>(acc, coef, B, L, loss_scale, grad_cutoff_dev,
                                                                        grad_q_dev, lane_loss);
  DGC_LAUNCHED(ctx, "biquad_bwd_final");
  sum_doubles_kernel<<<1, 32, 0, ctx->stream>>>(lane_loss, L, loss_dev);
  DGC_LAUNCHED(ctx, "biquad_loss_sum");
  return DGC_OK;
}

namespace {
// part[b][s] = sum over segment s of lam[n] * y[n-1] (n >= 1), in double
constexpr int OPG_SEGS = 32;
__global__ void __launch_bounds__(256)
onepole_ga_kernel(const float *__restrict__ lam, const float *__restrict__ y, int T, double *__restrict__ part) {
  const int b = blockIdx.y, sgm = blockIdx.x;
  const int64_t per = ((int64_t)T + OPG_SEGS - 1) / OPG_SEGS, lo = max((int64_t)1, sgm * per),
                hi = min((int64_t)T, (sgm + 1) * per);
  const float *lb = lam + (size_t)b * T, *yb = y + (size_t)b * T;
  double acc = 0.0;
  for (int64_t n = lo + threadIdx.x; n < hi; n += 256) acc += (double)lb[n] * (double)yb[n - 1];
  __shared__ double sh[256];
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) part[(size_t)b * OPG_SEGS + sgm] = sh[0];
}

__global__ void onepole_ga_sum_kernel(const double *__restrict__ part, int B, float *__restrict__ ga) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  double s = 0.0;
  for (int i = 0; i < OPG_SEGS; ++i) s += part[(size_t)b * OPG_SEGS + i];
  ga[b] = (float)s;
}
}  // namespace

// Backward of y[n] = x[n] + a y[n-1]: lam[n] = gy[n] + a lam[n+1] (the same scan, reversed in time),
// dL/dx = lam, dL/da[b] = sum_n lam[n] y[n-1].
DGC_EXPORT int32_t dgc_onepole_bwd(dgc_ctx *ctx, const float *y_dev, const float *gy_dev, int32_t B, int32_t T, float a,
                                   float *grad_x_dev, float *grad_a_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, gy_dev && grad_x_dev, "null pointer");
  DGC_REQUIRE(ctx, grad_a_dev == nullptr || y_dev != nullptr, "the coefficient gradient needs the forward output");
  DGC_REQUIRE(ctx, B > 0 && T > 0, "size out of range");
  DGC_REQUIRE(ctx, gy_dev != grad_x_dev, "in-place operation is not supported");
  const int NC = dgc_div_up(T, OP_CHUNK);
  DGC_REQUIRE(ctx, NC <= 65535 * 32 && B <= 65535, "size out of range");
  const uint64_t need = 2ull * B * NC + 2ull * B * OPG_SEGS + 8;
  float *scr = dgc_ctx_scratch(ctx, need);
  if (!scr) return DGC_ERR_OOM;
  float *chunk_end = scr, *carry = scr + (size_t)B * NC;
  double *part = reinterpret_cast<double *>(scr + (((size_t)2 * B * NC + 1) & ~(size_t)1));
  onepole_kernel<0, true><<<dim3(NC, B), OP_THREADS, 0, ctx->stream>>>(gy_dev, T, NC, a, nullptr, chunk_end, nullptr);
  DGC_LAUNCHED(ctx, "onepole_bwd_pass0");
  onepole_carry_kernel<<<dgc_div_up(B, 64), 64, 0, ctx->stream>>>(chunk_end, B, NC, a, 0.0f, carry);
  DGC_LAUNCHED(ctx, "onepole_bwd_carry");
  onepole_kernel<1, true><<<dim3(NC, B), OP_THREADS, 0, ctx->stream>>>(gy_dev, T, NC, a, carry, nullptr, grad_x_dev);
  DGC_LAUNCHED(ctx, "onepole_bwd_pass1");
  if (grad_a_dev) {
    onepole_ga_kernel<<<dim3(OPG_SEGS, B), 256, 0, ctx->stream>>>(grad_x_dev, y_dev, T, part);
    DGC_LAUNCHED(ctx, "onepole_grad_a");
    onepole_ga_sum_kernel<<<dgc_div_up(B, 128), 128, 0, ctx->stream>>>(part, B, grad_a_dev);
    DGC_LAUNCHED(ctx, "onepole_grad_a_sum");
  }
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_biquad_bwd(dgc_ctx *ctx, const dgc_biquad_params *p, const float *x_dev, const float *cutoff_dev,
                                  const float *q_dev, const float *y_dev, const float *gy_dev, float *scratch_dev,
                                  float *grad_cutoff_dev, float *grad_q_dev, float *grad_x_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, p && x_dev && cutoff_dev && q_dev && y_dev && gy_dev && grad_cutoff_dev && grad_q_dev,
              "null pointer");
  int32_t rc = biquad_validate(ctx, p);
  if (rc != DGC_OK) return rc;
  const int B = p->B, T = p->T, L = p->L, NC = dgc_div_up(T, BQ_CHUNK);
  DGC_REQUIRE(ctx, NC <= 65535, "T too large");
  float *scr = scratch_dev ? scratch_dev : dgc_ctx_scratch(ctx, dgc_biquad_scratch_floats(p, grad_x_dev ? 2 : 1));
  if (!scr) return DGC_ERR_OOM;
  DGC_REQUIRE(ctx, (((uintptr_t)scr) & 15) == 0, "scratch must be 16-byte aligned");
  float *coef = scr;
  float *rec = scr + ((((size_t)L * 24) + 3) & ~(size_t)3);
  size_t rec_n = ((size_t)B * NC * BW_REC * L + 3) & ~(size_t)3;
  double *acc = reinterpret_cast<double *>(rec + rec_n);
  double *lane_loss = acc + (size_t)B * L * 6;
  float *after = scr + dgc_biquad_scratch_floats(p, 1);
  float2 *term = grad_x_dev ? reinterpret_cast<float2 *>(after) : nullptr;
  float *part = after + (size_t)2 * B * NC * L;
  biquad_coef_kernel<<<dgc_div_up(L, 128), 128, 0, ctx->stream>>>(cutoff_dev, q_dev, L, p->gain, p->mode, coef);
  DGC_LAUNCHED(ctx, "biquad_coef");
  dim3 grid(dgc_div_up(L, BQ_THREADS), NC, B);
  biquad_bwd_kernel<true><<<grid, BQ_THREADS, 0, ctx->stream>>>(x_dev, coef, y_dev, gy_dev, B, T, L, NC, 1.0f, rec);
  DGC_LAUNCHED(ctx, "biquad_bwd");
  biquad_bwd_carry_kernel<<<dgc_div_up(B * L, 128), 128, 0, ctx->stream>>>(rec, coef, B, L, NC, T, acc, term);
  DGC_LAUNCHED(ctx, "biquad_bwd_carry");
  biquad_bwd_final_kernel<<<dgc_div_up(L, 128), 128, 0, ctx->stream>>>(acc, coef, B, L, 0.0f, grad_cutoff_dev, grad_q_dev,
                                                                        lane_loss);
  DGC_LAUNCHED(ctx, "biquad_bwd_final");
  if (grad_x_dev) {
    biquad_gx_kernel<true><<<grid, BQ_THREADS, 0, ctx->stream>>>(coef, y_dev, gy_dev, term, B, T, L, NC, 1.0f, part);
    DGC_LAUNCHED(ctx, "biquad_grad_x");
    const size_t n = (size_t)B * T;
    sum_partial_rows_kernel<<<dgc_div_up((int64_t)n, 256), 256, 0, ctx->stream>>>(part, (int)grid.x, n, grad_x_dev);
    DGC_LAUNCHED(ctx, "biquad_grad_x_sum");
  }
  return DGC_OK;
}

// ---------------------------------------------------------------------------------------------
// One-pole filter for callers that must not allocate.
//
// A real-time audio thread (a plug-in's render callback, a driver I/O thread) may not call anything
// that allocates or may block for an unbounded time; cudaMalloc does both, and a dgc_ctx allocates
// when it is created and whenever its scratch grows.  This entry point therefore takes no context:
// the chunk-carry scratch the scan needs lives in a fixed array in device memory that is part of the
// library image (every GPU that loads the library holds these 256 KiB until the process exits), and
// the caller supplies only the stream, the input and the output.
// ---------------------------------------------------------------------------------------------
#include <atomic>
#include <mutex>

namespace {
constexpr int STATIC_MAX_CHUNKS = DGC_ONEPOLE_STATIC_MAX_CHUNKS;
// [0, MAX): end value of every chunk; [MAX, 2 MAX): carry entering every chunk
static __device__ __align__(256) float g_onepole_static_scratch[2 * STATIC_MAX_CHUNKS];

constexpr int STATIC_MAX_DEVICES = 64;
// Resolved device address of the array, per device.  Published once with release ordering; every later call
// reads it with one acquire load and takes no lock, so a caller on a real-time thread never waits for another
// thread that is still in its own first call on some other device.
std::mutex g_static_mutex;   // serialises the one-time look-ups only
std::atomic<float *> g_static_ptr[STATIC_MAX_DEVICES];

void static_msg(char *buf, uint32_t len, const char *fmt, long long a = 0, long long b = 0) {
  if (buf && len) snprintf(buf, len, fmt, a, b);
}
}  // namespace

DGC_EXPORT int32_t dgc_onepole_fwd_static(void *cuda_stream, const float *x_dev, int32_t B, int32_t T, float a,
                                          float *y_dev, char *err_buf, uint32_t err_len) {
  if (err_buf && err_len) err_buf[0] = 0;
  if (!x_dev || !y_dev) {
    static_msg(err_buf, err_len, "dgc_onepole_fwd_static: null input or output pointer");
    return DGC_ERR_INVALID;
  }
  if (B <= 0 || T <= 0) {
    static_msg(err_buf, err_len, "dgc_onepole_fwd_static: B and T must be positive");
    return DGC_ERR_INVALID;
  }
  const long long NC = ((long long)T + OP_CHUNK - 1) / OP_CHUNK;
  if ((long long)B * NC > STATIC_MAX_CHUNKS || B > 65535) {
    static_msg(err_buf, err_len,
               "dgc_onepole_fwd_static: B*ceil(T/2048) = %lld exceeds the built-in scratch of %lld chunk slots; "
               "use dgc_onepole_fwd with a context for larger signals",
               (long long)B * NC, (long long)STATIC_MAX_CHUNKS);
    return DGC_ERR_INVALID;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= STATIC_MAX_DEVICES) {
    static_msg(err_buf, err_len, "dgc_onepole_fwd_static: no usable current device (cudaGetDevice = %lld)", (long long)e);
    return DGC_ERR_CUDA;
  }
  float *scratch = g_static_ptr[dev].load(std::memory_order_acquire);
  if (!scratch) {
    // Set-up, once per device, with that device current: the array's name is only a host-side
    // handle for the symbol; the address a kernel can use comes from cudaGetSymbolAddress.
    std::lock_guard<std::mutex> lock(g_static_mutex);
    scratch = g_static_ptr[dev].load(std::memory_order_relaxed);
    if (!scratch) {
      float *p = nullptr;
      e = cudaGetSymbolAddress((void **)&p, g_onepole_static_scratch);
      if (e != cudaSuccess || !p) {
        static_msg(err_buf, err_len, "dgc_onepole_fwd_static: cudaGetSymbolAddress failed (%lld) on device %lld",
                   (long long)e, (long long)dev);
        return DGC_ERR_CUDA;
      }
      g_static_ptr[dev].store(p, std::memory_order_release);
      scratch = p;
    }
  }
  // an error left behind by an unrelated earlier call must not be reported as a failure of these launches
  (void)cudaGetLastError();
  cudaStream_t st = (cudaStream_t)cuda_stream;
  float *chunk_end = scratch, *carry = scratch + STATIC_MAX_CHUNKS;
  // Every slot that is read below is written first by this call (chunk ends by pass 0, carries by the
  // carry kernel), so nothing has to be cleared although the array keeps the previous call's contents.
  onepole_kernel<0><<<dim3((unsigned)NC, B), OP_THREADS, 0, st>>>(x_dev, T, (int)NC, a, nullptr, chunk_end, nullptr);
  onepole_carry_kernel<<<dgc_div_up(B, 64), 64, 0, st>>>(chunk_end, B, (int)NC, a, 0.0f, carry);
  onepole_kernel<1><<<dim3((unsigned)NC, B), OP_THREADS, 0, st>>>(x_dev, T, (int)NC, a, carry, nullptr, y_dev);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    static_msg(err_buf, err_len, "dgc_onepole_fwd_static: launch failed (%lld)", (long long)e);
    return DGC_ERR_CUDA;
  }
  return DGC_OK;
}
