// Noise branch of the batched harmonic synth: a time-varying FIR whose taps are linearly
// interpolated between control rows at every sample (Examples/HarmonicE2E/Synth.swift:97-101),
// and the band-magnitude -> tap matrix product that feeds it in the synthetic workload.
#include <cstdlib>

#include "common.cuh"

namespace {

// Block = NTH threads, thread = SPT consecutive frames of one voice, tile = NTH*SPT frames.  NTH is picked by
// the host so that all blocks of the launch are resident at once (no second, mostly empty wave).
// Shared memory: the control rows the tile touches (R rows of `taps` floats) and the noise tile with
// its taps-1 frames of history, de-interleaved by (index mod SPT) so that the sliding window of a
// thread and of its neighbours falls in distinct banks.
// A thread's SPT frames see at most two (lo, hi) row pairs (the host guarantees step*SPT < 1), so it
// accumulates dot products against rows r0, r0+1 for every frame, and against r0+2 only when its
// frames straddle a control-row boundary.
template <int SPT, int NTH>
__global__ void __launch_bounds__(NTH, 4)
fir_noise_kernel(dgc_fir_params prm, const float2 *__restrict__ rowtab, const float *__restrict__ noise,
                 const float *__restrict__ taps_tab, const float *__restrict__ ngain, float *__restrict__ audio,
                 int max_rows, int32_t *status) {
  extern __shared__ float sh[];
  const int B = prm.B, T = prm.T, F = prm.F, NT = prm.taps;
  constexpr int TILE = NTH * SPT;
  const int b = blockIdx.y, t0 = blockIdx.x * TILE;
  const int t_last = min(T - 1, t0 + TILE - 1);
  // The control clock wraps to 0 when it reaches its maximum (the sequential single-precision
  // clock runs slightly fast, so this happens a few frames before the end of the render).  Find
  // the wrap frame of this tile, if any; row numbers after it are unwrapped (+F) so that the rows a
  // tile touches stay one contiguous run.
  __shared__ int wrap_sh;
  if (threadIdx.x == 0) wrap_sh = 0x7fffffff;
  __syncthreads();
#pragma unroll
  for (int u = 0; u < SPT; ++u) {
    int n = t0 + threadIdx.x * SPT + u;
    // (the cached row table holds the floor control row of every frame: a drop marks the wrap)
    if (n > t0 && n <= t_last && __float_as_int(rowtab[n].x) < __float_as_int(rowtab[n - 1].x)) atomicMin(&wrap_sh, n);
  }
  __syncthreads();
  const int wrap = wrap_sh;
  const int rmin = __float_as_int(rowtab[t0].x);
  int rmax = __float_as_int(rowtab[t_last].x);
  if (t_last >= wrap) rmax += F;
  const int R = rmax - rmin + 3;  // rows rmin .. rmax+2 (hi of the last frame, and the straddle row)
  if (R > max_rows) {
    if (threadIdx.x == 0) atomicExch(status, 101);  // control rate too high for the staged tile
    return;
  }
  float *rows = sh;                          // [R][NT]
  float *xs = sh + (size_t)max_rows * NT;    // [SPT][Q], Q = (TILE + NT - 1 + SPT - 1) / SPT + 1
  const int XN = TILE + NT - 1;
  const int Q = (XN + SPT - 1) / SPT + 1;
  {
    // flat copy of R * NT floats, independent iterations (the loads of several elements are in flight
    // together); i / NT by multiplication with ceil(2^32 / NT), exact for i * NT < 2^32
    const unsigned magic = (unsigned)((0x100000000ull + (unsigned)NT - 1) / (unsigned)NT);
#pragma unroll 4
    for (int i = threadIdx.x; i < R * NT; i += NTH) {
      const int rr = (int)__umulhi((unsigned)i, magic), col = i - rr * NT;
      int r = rmin + rr;
      if (r >= F) r -= F;  // the ceil row wraps to row 0
      if (r >= F) r = F - 1;
      rows[i] = taps_tab[((size_t)r * B + b) * NT + col];
    }
  }
  // xs position m <-> frame t0 - (NT-1) + m
  const float *xn = noise + (size_t)b * T;
  for (int m = threadIdx.x; m < XN; m += NTH) {
    int t = t0 - (NT - 1) + m;
    float v = (t >= 0 && t < T) ? xn[t] : 0.0f;
    xs[(m % SPT) * Q + m / SPT] = v;
  }
  __syncthreads();

  const int nl = threadIdx.x * SPT;  // first local frame of this thread
  if (t0 + nl >= T) return;
  int lo[SPT];
  float fr[SPT];
#pragma unroll
  for (int u = 0; u < SPT; ++u) {
    int n = min(t0 + nl + u, T - 1);
    const float2 rt = rowtab[n];
    lo[u] = __float_as_int(rt.x);
    fr[u] = rt.y;
    if (n >= wrap) lo[u] += F;
  }
  const int r0 = lo[0] - rmin;
  const int spread = lo[SPT - 1] - lo[0];
  const bool straddle = spread == 1;
  const float *ra = rows + (size_t)r0 * NT, *rb = ra + NT, *rc = rb + NT;
  float d0[SPT], d1[SPT], d2[SPT];
#pragma unroll
  for (int u = 0; u < SPT; ++u) d0[u] = d1[u] = d2[u] = 0.0f;

  // frame (nl+u), tap i reads xs position m = nl + u + i
  if (SPT == 8) {
    // Taps in groups of 8: W[0..15] holds x at positions nl + i0 .. nl + i0 + 15 (two shared-memory rows of the
    // de-interleaved tile per thread and group), so tap i0 + j of frame u multiplies W[u + j]: no per-tap
    // window rotation and no index arithmetic inside the 128 (256 with the second row) multiply-adds of a group.
    const float *xb = xs + threadIdx.x;   // W[t] = xb[(t % 8) * Q + i0 / 8 + t / 8]
    auto dots = [&](const float *pa, const float *pb, float(&e0)[SPT], float(&e1)[SPT], bool two) {
      float W[16];
#pragma unroll
      for (int t = 0; t < 8; ++t) W[t] = xb[t * Q];
      const int NG = NT / 8;
      for (int g8 = 0; g8 < NG; ++g8) {
#pragma unroll
        for (int t = 0; t < 8; ++t) W[8 + t] = xb[t * Q + g8 + 1];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float ta = pa[g8 * 8 + j];
#pragma unroll
          for (int u = 0; u < 8; ++u) e0[u] = fmaf(W[u + j], ta, e0[u]);
          if (two) {
            const float tb = pb[g8 * 8 + j];
#pragma unroll
            for (int u = 0; u < 8; ++u) e1[u] = fmaf(W[u + j], tb, e1[u]);
          }
        }
#pragma unroll
        for (int t = 0; t < 8; ++t) W[t] = W[8 + t];
      }
      // remaining taps (NT % 8), W[0..7] = positions nl + 8 * NG ..
      const int rem = NT - NG * 8;
      if (rem > 0) {
#pragma unroll
        for (int t = 0; t < 8; ++t) W[8 + t] = xb[t * Q + NG + 1];
#pragma unroll
        for (int j = 0; j < 7; ++j) {
          if (j < rem) {
            const float ta = pa[NG * 8 + j];
#pragma unroll
            for (int u = 0; u < 8; ++u) e0[u] = fmaf(W[u + j], ta, e0[u]);
            if (two) {
              const float tb = pb[NG * 8 + j];
#pragma unroll
              for (int u = 0; u < 8; ++u) e1[u] = fmaf(W[u + j], tb, e1[u]);
            }
          }
        }
      }
    };
    dots(ra, rb, d0, d1, true);
    if (straddle) dots(rc, rc, d2, d2, false);
  } else {
  float win[SPT];
#pragma unroll
  for (int u = 0; u < SPT - 1; ++u) win[u + 1] = xs[((nl + u) % SPT) * Q + (nl + u) / SPT];
  for (int i = 0; i < NT; ++i) {
#pragma unroll
    for (int u = 0; u < SPT - 1; ++u) win[u] = win[u + 1];
    {
      int m = nl + SPT - 1 + i;
      win[SPT - 1] = xs[(m % SPT) * Q + m / SPT];
    }
    float ta = ra[i], tb = rb[i];
#pragma unroll
    for (int u = 0; u < SPT; ++u) {
      d0[u] = fmaf(win[u], ta, d0[u]);
      d1[u] = fmaf(win[u], tb, d1[u]);
    }
  }
  if (straddle) {
#pragma unroll
    for (int u = 0; u < SPT - 1; ++u) win[u + 1] = xs[((nl + u) % SPT) * Q + (nl + u) / SPT];
    for (int i = 0; i < NT; ++i) {
#pragma unroll
      for (int u = 0; u < SPT - 1; ++u) win[u] = win[u + 1];
      int m = nl + SPT - 1 + i;
      win[SPT - 1] = xs[(m % SPT) * Q + m / SPT];
      float tc = rc[i];
#pragma unroll
      for (int u = 0; u < SPT; ++u) d2[u] = fmaf(win[u], tc, d2[u]);
    }
  }
  }
  if (spread > 1 || spread < 0) {
    // the frames of this thread sit across the clock wrap: evaluate each frame against its own rows
#pragma unroll
    for (int u = 0; u < SPT; ++u) {
      const float *pa = rows + (size_t)(lo[u] - rmin) * NT, *pb = pa + NT;
      float sa = 0.0f, sb = 0.0f;
      for (int i = 0; i < NT; ++i) {
        int m = nl + u + i;
        float xv = xs[(m % SPT) * Q + m / SPT];
        sa = fmaf(xv, pa[i], sa);
        sb = fmaf(xv, pb[i], sb);
      }
      d0[u] = sa;
      d1[u] = sb;
    }
  }
  float *dst = audio + (size_t)b * T;
#pragma unroll
  for (int u = 0; u < SPT; ++u) {
    int n = t0 + nl + u;
    if (n >= T) break;
    bool second = straddle && lo[u] != lo[0];
    float a = second ? d1[u] : d0[u], c = second ? d2[u] : d1[u];
    float omf = 1.0f - fr[u];
    int l = lo[u] >= F ? lo[u] - F : lo[u], h = l + 1 >= F ? 0 : l + 1;
    float ng = fmaf(fr[u], ngain[(size_t)h * B + b], omf * ngain[(size_t)l * B + b]);
    float y = fmaf(fr[u], c, omf * a) * ng * prm.scale;
    dst[n] = prm.accumulate ? dst[n] + y : y;
  }
}

// The same filter with the shared-memory traffic and the third dot product taken out of the main loop.
//   * control rows are staged with a padded stride NTP (a multiple of 4 with NTP % 8 == 4, zero beyond `taps`):
//     a thread reads four taps of a row with ONE 128-bit load (rows of the four 8-lane groups of a warp fall into
//     distinct bank quads), so eight taps x two rows x eight frames = 128 multiply-adds cost 4 tap loads and 8 signal
//     loads; no remainder loop (the padding taps are zero, the signal tile is zero-extended to match);
//   * a thread whose eight frames straddle a control-row boundary needs a third row for the frames behind the
//     boundary.  Computed inside the main loop that third dot product makes EVERY warp run the loop body a third
//     time for its few straddling lanes (+50 % instructions).  Here the straddling threads put themselves on a
//     list, and after the main loop every group of 8 lanes takes one list entry: the lanes split the taps, slide
//     the signal window through registers, and reduce with shuffles (+9 % instructions).
// Block = NTH threads x 8 frames.  Results are bit-identical from run to run (fixed summation orders; the list
// order only decides which lane group computes an entry, not how).
// RB: resident blocks per SM the registers are capped for (0: 768 threads for 8 frames per thread, 512 for 16).
template <int NTH, int SPT, int RB = 0>
__global__ void __launch_bounds__(NTH, RB ? RB : (SPT == 8 ? 768 : 512) / NTH)
fir_noise8_kernel(dgc_fir_params prm, const float2 *__restrict__ rowtab, const float *__restrict__ noise,
                  const float *__restrict__ taps_tab, const float *__restrict__ ngain, float *__restrict__ audio,
                  int max_rows, int NTP, int32_t *status) {
  extern __shared__ __align__(16) float sh[];
  constexpr int TILE = NTH * SPT, GROUPS = NTH / 8;
  const int B = prm.B, T = prm.T, F = prm.F, NT = prm.taps;
  const int b = blockIdx.y, t0 = blockIdx.x * TILE;
  const int t_last = min(T - 1, t0 + TILE - 1);
  __shared__ int n_list;               // straddling threads: their list and third dot products live behind the tile
  // Threads whose frames sit across the clock wrap (the row numbers jump there: each frame has its own pair of
  // rows).  At most one per tile while the playhead sweeps the rows once; the whole block evaluates them together
  // after the main loop -- left to the thread itself, those 8 x 2 x taps dependent multiply-adds keep one block
  // (and the SM that hosts it) busy for as long again as the rest of the tile.
  constexpr int IRR_MAX = 4, PARTS = NTH / SPT;
  __shared__ int n_irr, irr_list[IRR_MAX];
  __shared__ float irr_buf[IRR_MAX][SPT][2];
  if (threadIdx.x == 0) {
    n_list = 0;
    n_irr = 0;
  }
  // The frame at which the control clock wrapped (entry T of the row table; above every frame when it never does:
  // the playhead sweeps the control rows once, so there is at most one).  It concerns this tile only when it lies
  // strictly inside: the rows behind it are then numbered F, F + 1, .. so that the tile's rows stay ascending.
  const int wrap_all = __float_as_int(rowtab[T].x);
  const int wrap = (wrap_all > t0 && wrap_all <= t_last) ? wrap_all : 0x7fffffff;
  const int rmin = __float_as_int(rowtab[t0].x);
  int rmax = __float_as_int(rowtab[t_last].x);
  if (t_last >= wrap) rmax += F;
  const int R = rmax - rmin + 3;  // rows rmin .. rmax+2 (hi of the last frame, and the straddle row)
  if (R > max_rows) {
    if (threadIdx.x == 0) atomicExch(status, 101);  // control rate too high for the staged tile
    return;
  }
  float *rows = sh;                          // [R][NTP]
  float *xs = sh + (size_t)max_rows * NTP;   // [SPT][Q]: position m <-> frame t0 - (NT-1) + m, de-interleaved by m % SPT
  const int XN = TILE + NTP - 1 + SPT;       // zero-extended: the padding taps read beyond the tile
  const int Q = (XN + SPT - 1) / SPT + 1;
  // every control-row boundary inside the tile makes one thread straddle: at most max_rows entries
  float *d2buf = xs + (size_t)SPT * Q;                               // [max_rows][SPT], by list position
  int *list = reinterpret_cast<int *>(d2buf + (size_t)max_rows * SPT);   // [max_rows]
  // Staging by asynchronous 4-byte copies (the rows of the tap table are not 16-byte aligned): every copy of the
  // tile is in flight before the first one is waited for, and nothing passes through registers.  One warp per
  // control row, lanes along the taps (coalesced, no index division); padding taps and frames outside the signal
  // are zero-filled by the copy itself (source size 0).
  for (int rr = threadIdx.x >> 5; rr < R; rr += NTH / 32) {
    int r = rmin + rr;
    if (r >= F) r -= F;  // the ceil row wraps to row 0
    if (r >= F) r = F - 1;
    const float *src = taps_tab + ((size_t)r * B + b) * NT;
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(rows + (size_t)rr * NTP);
    for (int col = threadIdx.x & 31; col < NTP; col += 32) {
      const bool in = col < NT;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst + 4u * col), "l"(in ? src + col : src),
                   "r"(in ? 4 : 0)
                   : "memory");
    }
  }
  const float *xn = noise + (size_t)b * T;
  for (int m = threadIdx.x; m < Q * SPT; m += NTH) {
    const int t = t0 - (NT - 1) + m;
    const bool in = t >= 0 && t < T && m < TILE + NT - 1;
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(xs + (m & (SPT - 1)) * Q + m / SPT);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(in ? xn + t : xn), "r"(in ? 4 : 0)
                 : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  const int nl = threadIdx.x * SPT;  // first local frame of this thread
  const bool have = t0 + nl < T;
  int lo[SPT];
  float fr[SPT];
#pragma unroll
  for (int u = 0; u < SPT; ++u) {
    int n = min(t0 + nl + u, T - 1);
    const float2 rt = rowtab[n];
    lo[u] = __float_as_int(rt.x);
    fr[u] = rt.y;
    if (n >= wrap) lo[u] += F;
  }
  const int r0 = lo[0] - rmin;
  const int spread = lo[SPT - 1] - lo[0];
  const bool straddle = have && spread == 1;
  float d0[SPT], d1[SPT], d2[SPT];
#pragma unroll
  for (int u = 0; u < SPT; ++u) d0[u] = d1[u] = d2[u] = 0.0f;
  int my_entry = -1;
  bool overflow = false;   // more straddling threads than the list holds (cannot happen while rows ascend): slow path
  if (straddle) {
    my_entry = atomicAdd(&n_list, 1);
    if (my_entry < max_rows) list[my_entry] = threadIdx.x;
    else {
      overflow = true;
      my_entry = -1;
    }
  }
  int my_irr = -1;
  if (have && (spread > 1 || spread < 0 || overflow)) {
    my_irr = atomicAdd(&n_irr, 1);
    if (my_irr < IRR_MAX) irr_list[my_irr] = threadIdx.x;
  }
  if (have) {
    // frame (nl+u), tap i reads xs position nl + u + i; W[w] = position nl + SPT g + w = xb[(w % SPT) * Q + g + w / SPT]
    const float4 *pa = reinterpret_cast<const float4 *>(rows + (size_t)r0 * NTP);
    const float4 *pb = reinterpret_cast<const float4 *>(rows + (size_t)(r0 + 1) * NTP);
    const float *xb = xs + threadIdx.x;
    float W[2 * SPT];
#pragma unroll
    for (int t = 0; t < SPT; ++t) W[t] = xb[t * Q];
    const int NG = NTP / SPT, rem = NTP - NG * SPT;     // rem: 4 (SPT 8), 4 or 12 (SPT 16)
    auto four = [&](const float4 ta, const float4 tb, int j0) {
      const float a[4] = {ta.x, ta.y, ta.z, ta.w}, c[4] = {tb.x, tb.y, tb.z, tb.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int u = 0; u < SPT; ++u) {
          d0[u] = fmaf(W[u + j0 + j], a[j], d0[u]);
          d1[u] = fmaf(W[u + j0 + j], c[j], d1[u]);
        }
    };
#pragma unroll(SPT == 8 ? 4 : 2)
    for (int g = 0; g < NG; ++g) {
#pragma unroll
      for (int t = 0; t < SPT; ++t) W[SPT + t] = xb[t * Q + g + 1];
#pragma unroll
      for (int jb = 0; jb < SPT / 4; ++jb) four(pa[g * (SPT / 4) + jb], pb[g * (SPT / 4) + jb], 4 * jb);
#pragma unroll
      for (int t = 0; t < SPT; ++t) W[t] = W[SPT + t];
    }
#pragma unroll
    for (int t = 0; t < SPT - 4; ++t) W[SPT + t] = t < rem ? xb[t * Q + NG + 1] : 0.0f;
#pragma unroll
    for (int jb = 0; jb < SPT / 4 - 1; ++jb)
      if (4 * jb < rem) four(pa[NG * (SPT / 4) + jb], pb[NG * (SPT / 4) + jb], 4 * jb);
  }
  __syncthreads();
  // third rows of the straddling threads: one list entry per group of 8 lanes, lanes split the taps
  {
    const int grp = threadIdx.x >> 3, l8 = threadIdx.x & 7;
    const unsigned gmask = 0xffu << (8 * (grp & 3));   // the 8 lanes of this group (trip counts differ between groups)
    const int per = (NTP + 7) / 8;
    const int nent = min(n_list, max_rows);
    for (int e = grp; e < nent; e += GROUPS) {
      const int th = list[e];
      const int nls = th * SPT;
      // the entry thread's r0: floor row of its first frame
      const int n_first = min(t0 + nls, T - 1);
      int lo0 = __float_as_int(rowtab[n_first].x);
      if (n_first >= wrap) lo0 += F;
      const float *rc = rows + (size_t)(lo0 - rmin + 2) * NTP;
      const int i0 = l8 * per, i1 = min(NTP, i0 + per);
      float acc[SPT], Wd[SPT];
#pragma unroll
      for (int u = 0; u < SPT; ++u) acc[u] = 0.0f;
#pragma unroll
      for (int u = 0; u < SPT - 1; ++u) {
        const int m = nls + u + i0;
        Wd[u + 1] = xs[(m % SPT) * Q + m / SPT];
      }
      for (int i = i0; i < i1; ++i) {
#pragma unroll
        for (int u = 0; u < SPT - 1; ++u) Wd[u] = Wd[u + 1];
        const int m = nls + SPT - 1 + i;
        Wd[SPT - 1] = xs[(m % SPT) * Q + m / SPT];
        const float tc = rc[i];
#pragma unroll
        for (int u = 0; u < SPT; ++u) acc[u] = fmaf(Wd[u], tc, acc[u]);
      }
#pragma unroll
      for (int u = 0; u < SPT; ++u) {
        float v = acc[u];
        v += __shfl_xor_sync(gmask, v, 1);
        v += __shfl_xor_sync(gmask, v, 2);
        v += __shfl_xor_sync(gmask, v, 4);
        if (l8 == 0) d2buf[e * SPT + u] = v;
      }
    }
  }
  // irregular threads: thread (u, part) of the block takes frame u of the entry and every PARTS-th tap
  {
    const int nirr = min(n_irr, IRR_MAX);
    const int u = threadIdx.x / PARTS, part = threadIdx.x % PARTS;
    for (int e = 0; e < nirr; ++e) {
      const int nls = irr_list[e] * SPT;
      const int n = min(t0 + nls + u, T - 1);
      int lo_u = __float_as_int(rowtab[n].x);
      if (n >= wrap) lo_u += F;
      const float *pa = rows + (size_t)(lo_u - rmin) * NTP, *pb = pa + NTP;
      float sa = 0.0f, sb = 0.0f;
      for (int i = part; i < NT; i += PARTS) {
        const int m = nls + u + i;
        const float xv = xs[(m % SPT) * Q + m / SPT];
        sa = fmaf(xv, pa[i], sa);
        sb = fmaf(xv, pb[i], sb);
      }
#pragma unroll
      for (int off = PARTS / 2; off > 0; off >>= 1) {
        sa += __shfl_xor_sync(0xffffffffu, sa, off);
        sb += __shfl_xor_sync(0xffffffffu, sb, off);
      }
      if (part == 0) {
        irr_buf[e][u][0] = sa;
        irr_buf[e][u][1] = sb;
      }
    }
  }
  __syncthreads();
  if (!have) return;
  if (my_entry >= 0) {
#pragma unroll
    for (int u = 0; u < SPT; ++u) d2[u] = d2buf[my_entry * SPT + u];
  }
  if (my_irr >= 0 && my_irr < IRR_MAX) {
#pragma unroll
    for (int u = 0; u < SPT; ++u) {
      d0[u] = irr_buf[my_irr][u][0];
      d1[u] = irr_buf[my_irr][u][1];
    }
  } else if (my_irr >= 0) {
    // more irregular threads than the block-wide pass takes: evaluate each frame against its own rows here
#pragma unroll
    for (int u = 0; u < SPT; ++u) {
      const float *pa = rows + (size_t)(lo[u] - rmin) * NTP, *pb = pa + NTP;
      float sa = 0.0f, sb = 0.0f;
      for (int i = 0; i < NT; ++i) {
        int m = nl + u + i;
        float xv = xs[(m % SPT) * Q + m / SPT];
        sa = fmaf(xv, pa[i], sa);
        sb = fmaf(xv, pb[i], sb);
      }
      d0[u] = sa;
      d1[u] = sb;
    }
  }
  float *dst = audio + (size_t)b * T;
#pragma unroll
  for (int u = 0; u < SPT; ++u) {
    int n = t0 + nl + u;
    if (n >= T) break;
    bool second = straddle && my_irr < 0 && lo[u] != lo[0];
    float a = second ? d1[u] : d0[u], c = second ? d2[u] : d1[u];
    float omf = 1.0f - fr[u];
    int l = lo[u] >= F ? lo[u] - F : lo[u], h = l + 1 >= F ? 0 : l + 1;
    float ng = fmaf(fr[u], ngain[(size_t)h * B + b], omf * ngain[(size_t)l * B + b]);
    float y = fmaf(fr[u], c, omf * a) * ng * prm.scale;
    dst[n] = prm.accumulate ? dst[n] + y : y;
  }
}

// The band -> tap map as a plain single-precision tile kernel: C[M][N] = A[M][K] * W[N][K]^T with a SHORT reduction
// (K = 65 bands) and a wide output (N = 257 taps), shaped for the case: both 128-row operand tiles sit WHOLE in
// shared memory, row-major as they lie in global memory (rows of KS floats, KS % 8 == 4, zero beyond K), staged
// once by 4-byte asynchronous copies (a warp per row, lanes along k: coalesced), one barrier, then the reduction
// four k values at a time: a thread owns an 8 x 8 register tile of interleaved rows and columns, so that the
// lanes of a warp read eight consecutive rows of A and four consecutive rows of W as conflict-free 16-byte
// fragments along k (16 loads per 256 multiply-adds).  Exact single-precision accumulation in k order.
// A remainder of at most TMAP_NARROW columns (N = 257 = 2 x 128 + 1) is computed by the last tile's block as dot
// products: blocks of their own for it made the 16-voice grid 1.27 waves.
constexpr int TMAP_KMAX = 80, TMAP_NARROW = 16;
// row length of the staged tiles: the smallest multiple of 4 at or above K that is 4 modulo 8
__host__ __device__ constexpr int tmap_stride(int K) { return ((K + 3) & ~3) % 8 == 4 ? ((K + 3) & ~3) : ((K + 3) & ~3) + 4; }

__global__ void __launch_bounds__(256, 2)
tap_map_tile_kernel(const float *__restrict__ A, const float *__restrict__ W, int M, int N, int K, float *__restrict__ C) {
  extern __shared__ __align__(16) float tmap_sh[];
  const int tid = threadIdx.x, m0 = blockIdx.y * 128, n0 = blockIdx.x * 128;
  // columns of this tile; a remainder of at most TMAP_NARROW columns behind the last full tile (N = 257 = 2 x 128 + 1)
  // is not worth blocks of its own: the last tile's block computes it as dot products after its main loop
  const int nw = min(128, N - n0);
  const int extra = (blockIdx.x == gridDim.x - 1) ? N - n0 - nw : 0;
  // Both tiles row-major as they lie in memory, rows of KS floats with KS % 8 == 4 (16-byte aligned rows whose
  // starts fall into bank quads 4 apart), zero beyond K.  Staged by 4-byte asynchronous copies, one warp per row
  // with the lanes along k: coalesced global reads, consecutive shared-memory writes.
  const int KS = tmap_stride(K);
  float *As = tmap_sh, *Ws = tmap_sh + 128 * KS;
  const int warp = tid >> 5, lane = tid & 31;
  {
    const uint32_t as = (uint32_t)__cvta_generic_to_shared(As), ws = (uint32_t)__cvta_generic_to_shared(Ws);
    for (int r = warp; r < 128; r += 8) {
      const bool ina = m0 + r < M, inw = n0 + r < N;
      const float *ga = A + (size_t)(ina ? m0 + r : 0) * K, *gw = W + (size_t)(inw ? n0 + r : 0) * K;
      for (int k = lane; k < KS; k += 32) {
        const bool ink = k < K;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(as + 4u * (r * KS + k)),
                     "l"(ink ? ga + k : ga), "r"(ina && ink ? 4 : 0)
                     : "memory");
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(ws + 4u * (r * KS + k)),
                     "l"(ink ? gw + k : gw), "r"(inw && ink ? 4 : 0)
                     : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }
  __syncthreads();
  // 2 x 4 warps of 64 x 32 outputs, 8 x 4 lanes; a thread owns the rows wm + ly + 8 i and the columns wn + lx + 4 j
  // (i, j < 8): for a fixed i the eight ly lanes read eight CONSECUTIVE rows, whose 16-byte fragments along k sit in
  // eight different bank quads -- so both operands are read four k values at a time with one conflict-free
  // 16-byte load each: 16 loads per 256 multiply-adds.
  const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
  const int ly = lane >> 2, lx = lane & 3;
  const float *ap = As + (wm + ly) * KS, *bp = Ws + (wn + lx) * KS;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
#pragma unroll 1
  for (int k = 0; k < KS; k += 4) {
    float4 a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = *reinterpret_cast<const float4 *>(ap + (8 * i) * KS + k);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 b = *reinterpret_cast<const float4 *>(bp + (4 * j) * KS + k);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        acc[i][j] = fmaf(a[i].x, b.x, acc[i][j]);
        acc[i][j] = fmaf(a[i].y, b.y, acc[i][j]);
        acc[i][j] = fmaf(a[i].z, b.z, acc[i][j]);
        acc[i][j] = fmaf(a[i].w, b.w, acc[i][j]);
      }
    }
  }
  // the remainder columns: thread (row, column) pairs, the A row from shared memory, the W row from global memory
  for (int idx = tid; idx < 128 * extra; idx += 256) {
    const int m = idx % 128, c = idx / 128;
    if (m0 + m >= M) continue;
    const float *a = As + m * KS, *w = W + (size_t)(n0 + 128 + c) * K;
    float sum = 0.0f;
    for (int k = 0; k < K; ++k) sum = fmaf(a[k], __ldg(w + k), sum);
    C[(size_t)(m0 + m) * N + n0 + 128 + c] = sum;
  }
  // The tile leaves through shared memory (the operand tiles are done with): a thread's 8 x 8 outputs are scattered
  // over 8 rows and 8 columns, so storing them directly would write 16-byte pieces of 8 different rows per
  // instruction; from the staged tile a warp writes whole rows, 128 contiguous bytes per instruction.
  __syncthreads();
  float *Cs = tmap_sh;                       // [128][132]: 132 % 32 == 4, the 8 x 4 lanes of a store hit 32 banks
  constexpr int LDC = 132;
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) Cs[(wm + ly + 8 * i) * LDC + wn + lx + 4 * j] = acc[i][j];
  __syncthreads();
  for (int r = warp; r < 128; r += 8) {
    const int gm = m0 + r;
    if (gm >= M) break;
    float *row = C + (size_t)gm * N + n0;
    for (int c = lane; c < nw; c += 32) row[c] = Cs[r * LDC + c];
  }
}

// taps[r][i] = sum_j W[i][j] * bands[r][j]; W is staged once per block and reused for BT_PASSES
// groups of 16 rows; thread = taps i, i+256, ...
constexpr int BT_PASSES = 8;

__global__ void __launch_bounds__(256)
bands_to_taps_kernel(const float *__restrict__ bands, const float *__restrict__ w, int rows, int nb, int nt,
                     float *__restrict__ out) {
  extern __shared__ float sh[];
  const int ws = nb | 1;                 // odd row stride: conflict-free column walks
  float *wsh = sh;                       // [nt][ws]
  float *bsh = sh + (((size_t)nt * ws + 3) & ~(size_t)3);  // [nb][16], row index fastest, 16-byte aligned
  for (int i = threadIdx.x; i < nt * nb; i += 256) wsh[(i / nb) * ws + (i % nb)] = w[i];
  for (int pass = 0; pass < BT_PASSES; ++pass) {
    const int r0 = (blockIdx.x * BT_PASSES + pass) * 16;
    if (r0 >= rows) break;
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * nb; i += 256) {
      int r = i / nb, j = i - r * nb;
      bsh[j * 16 + r] = (r0 + r < rows) ? bands[(size_t)(r0 + r) * nb + j] : 0.0f;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nt; i += 256) {
      float acc[16];
#pragma unroll
      for (int r = 0; r < 16; ++r) acc[r] = 0.0f;
      const float *wr = wsh + (size_t)i * ws;
      for (int j = 0; j < nb; ++j) {
        float wv = wr[j];
        const float4 *bp = reinterpret_cast<const float4 *>(bsh + j * 16);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float4 v = bp[q];
          acc[4 * q + 0] = fmaf(wv, v.x, acc[4 * q + 0]);
          acc[4 * q + 1] = fmaf(wv, v.y, acc[4 * q + 1]);
          acc[4 * q + 2] = fmaf(wv, v.z, acc[4 * q + 2]);
          acc[4 * q + 3] = fmaf(wv, v.w, acc[4 * q + 3]);
        }
      }
#pragma unroll
      for (int r = 0; r < 16; ++r)
        if (r0 + r < rows) out[(size_t)(r0 + r) * nt + i] = acc[r];
    }
  }
}

}  // namespace

DGC_EXPORT int32_t dgc_fir_noise(dgc_ctx *ctx, const dgc_fir_params *p, const float *noise_dev,
                                 const float *taps_dev, const float *noise_gain_dev, float *audio_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, p && noise_dev && taps_dev && noise_gain_dev && audio_dev, "null pointer");
  DGC_REQUIRE(ctx, p->B > 0 && p->T > 0 && p->F > 0, "size out of range");
  DGC_REQUIRE(ctx, p->taps >= 1 && p->taps <= 1024, "taps must be in 1..1024");
  const float2 *play = dgc_ctx_row_table(ctx, p->F, p->T);   // (floor row, fraction) of every frame
  if (!play) return DGC_ERR_CUDA;
  int32_t rc = DGC_OK;
  // playhead advance per frame; the sequential single-precision clock runs up to ~0.5% fast
  double step = p->T > 1 ? (double)(p->F - 1) / (double)(p->T - 1) : 0.0;
  step *= 1.01;
  const int NT = p->taps;
  auto launch = [&](auto kern, int spt, int nth) -> int32_t {
    int tile = nth * spt;
    int max_rows = (int)(step * tile) + 5;
    size_t smem = ((size_t)max_rows * NT + (size_t)spt * ((tile + NT - 1 + spt - 1) / spt + 1)) * sizeof(float);
    if (smem > 200 * 1024) return DGC_ERR_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return dgc_fail(ctx, DGC_ERR_CUDA, "fir smem opt-in: %s", cudaGetErrorString(e));
    kern<<<dim3(dgc_div_up(p->T, tile), p->B), nth, smem, ctx->stream>>>(*p, play, noise_dev, taps_dev,
                                                                          noise_gain_dev, audio_dev, max_rows,
                                                                          ctx->status_dev);
    ctx->launches++;
    return dgc_check_launch(ctx, "fir_noise");
  };
  rc = DGC_ERR_UNSUPPORTED;
  static const int fir_variant = [] {
    const char *e = getenv("DGC_FIR");
    return e ? atoi(e) : 128;           // threads per block of the list-based kernel; 0 = the in-loop variant
  }();
  // frames per thread of the list-based kernel.  16 (DGC_FIR_SPT=16) halves the shared-memory traffic per
  // multiply-add (16 new signal values and 16 taps of two rows feed 512 multiply-adds instead of 128 for 8 and 8),
  // but its 128 registers per thread cost more in resident warps than the traffic saves: measured 0.78 ms against
  // 0.59 ms for 8 frames per thread at 256 voices, 0.097 against 0.076 ms at 16
  static const int fir_spt = [] {
    const char *e = getenv("DGC_FIR_SPT");
    return e && atoi(e) == 16 ? 16 : 8;
  }();
  const int spt = (fir_spt == 16 && step * 16 < 0.98 && NT >= 16) ? 16 : 8;
  if (step * 8 < 0.98 && fir_variant > 0) {
    int NTP = (NT + 3) & ~3;
    if (NTP % 8 == 0) NTP += 4;
    auto launch8 = [&](auto kern, int nth) -> int32_t {
      const int tile = nth * spt;
      const int max_rows = (int)(step * tile) + 5;
      const int XN = tile + NTP - 1 + spt, Q = (XN + spt - 1) / spt + 1;
      const size_t smem = ((size_t)max_rows * NTP + (size_t)spt * Q + (size_t)max_rows * (spt + 1)) * sizeof(float);
      if (smem > 160 * 1024) return DGC_ERR_UNSUPPORTED;
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return dgc_fail(ctx, DGC_ERR_CUDA, "fir smem opt-in: %s", cudaGetErrorString(e));
      kern<<<dim3(dgc_div_up(p->T, tile), p->B), nth, smem, ctx->stream>>>(*p, play, noise_dev, taps_dev, noise_gain_dev,
                                                                            audio_dev, max_rows, NTP, ctx->status_dev);
      ctx->launches++;
      return dgc_check_launch(ctx, "fir_noise8");
    };
    if (spt == 16) rc = fir_variant == 64 ? launch8(fir_noise8_kernel<64, 16>, 64) : launch8(fir_noise8_kernel<128, 16>, 128);
    else if (fir_variant == 256) rc = launch8(fir_noise8_kernel<256, 8>, 256);
    else {
      // A grid that fits 7 resident blocks per SM but not 6 (16 voices x 64000 frames: 1008 blocks on 148 SMs) runs
      // as ONE wave on the 72-register build instead of a full wave and a nearly empty second one (the per-SM busy
      // time of that launch was 58k to 120k cycles: half the SMs idle for half the kernel).  Larger grids keep the
      // 80-register build, which is 3 % faster per block.
      const int64_t nblocks = (int64_t)dgc_div_up(p->T, 128 * 8) * p->B;
      if (nblocks > 6 * (int64_t)ctx->sm_count && nblocks <= 7 * (int64_t)ctx->sm_count) {
        cudaFuncSetAttribute(fir_noise8_kernel<128, 8, 7>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        rc = launch8(fir_noise8_kernel<128, 8, 7>, 128);
      } else
        rc = launch8(fir_noise8_kernel<128, 8>, 128);
    }
  }
  if (rc == DGC_ERR_UNSUPPORTED && step * 8 < 0.98) {
    // 256-thread tiles amortise the staged control rows best (measured against 128 and 64 at the headline
    // configuration: 82.5 / 86.5 / 83 us); DGC_FIR_THREADS forces a tile size for experiments
    static const int forced = [] {
      const char *e = getenv("DGC_FIR_THREADS");
      return e ? atoi(e) : 0;
    }();
    int nth = 256;
    if (forced == 64 || forced == 128 || forced == 256) nth = forced;
    if (nth == 256) rc = launch(fir_noise_kernel<8, 256>, 8, 256);
    else if (nth == 128) rc = launch(fir_noise_kernel<8, 128>, 8, 128);
    else rc = launch(fir_noise_kernel<8, 64>, 8, 64);
  }
  if (rc == DGC_ERR_UNSUPPORTED) rc = launch(fir_noise_kernel<1, 256>, 1, 256);
  if (rc == DGC_ERR_UNSUPPORTED)
    return dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "fir_noise: control rate too high for the shared-memory tile");
  return rc;
}

DGC_EXPORT int32_t dgc_bands_to_taps(dgc_ctx *ctx, const float *bands_dev, const float *w_dev, int32_t rows,
                                     int32_t nbands, int32_t taps, float *taps_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, bands_dev && w_dev && taps_dev, "null pointer");
  DGC_REQUIRE(ctx, rows > 0 && nbands > 0 && taps > 0, "size out of range");
  // From 2^24 multiply-adds on the map runs as a matmul.  For 32 to 72 bands and at least 128 taps: the persistent
  // short-reduction tensor-core kernel of the matmul entry point (3xTF32 with rounded parts; a CTA keeps its 128
  // taps of the matrix in shared memory and streams row tiles of the bands through two accumulators): 17 us for
  // the 16-voice map and 0.124 ms for the 256-voice one under the profiler, against 28 us and 0.32 ms for the plain
  // fp32 tile kernel and 0.30 ms for the general tensor-core pipeline; whole steps 0.166 against 0.172 ms (16
  // voices) and 2.15 against 2.32 ms (256).  Other shapes: the tile kernel up to 1024 output tiles, the matmul entry point beyond.
  // DGC_TAP_MAP=tile|tc forces the tile kernel / the matmul entry point.
  const char *tmap_env = getenv("DGC_TAP_MAP");   // read per call: a test can switch kernels inside one process
  const int tmap_mode = !tmap_env ? 0 : strcmp(tmap_env, "tc") == 0 ? 1 : strcmp(tmap_env, "tile") == 0 ? 2 : 0;
  const bool big = (double)rows * nbands * taps >= (double)(1 << 24);
  if (big && tmap_mode != 2 && dgc_gemm_nt_persistent(ctx, bands_dev, rows, taps, nbands))
    return dgc_gemm_nt(ctx, bands_dev, w_dev, rows, taps, nbands, taps_dev);
  const bool tmap_tile = tmap_mode == 2 || (tmap_mode == 0 && (int64_t)dgc_div_up(rows, 128) * dgc_div_up(taps, 128) <= 1024);
  if ((double)rows * nbands * taps >= (double)(1 << 24) && nbands <= TMAP_KMAX && tmap_tile) {
    size_t smem = (size_t)2 * 128 * tmap_stride(nbands) * sizeof(float);
    if (smem < (size_t)128 * 132 * sizeof(float)) smem = (size_t)128 * 132 * sizeof(float);   // the staged output tile
    DGC_CUDA(ctx, cudaFuncSetAttribute(tap_map_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int rem = taps % 128;
    const int ntx = (taps >= 128 && rem > 0 && rem <= TMAP_NARROW) ? taps / 128 : dgc_div_up(taps, 128);
    tap_map_tile_kernel<<<dim3(ntx, dgc_div_up(rows, 128)), 256, smem, ctx->stream>>>(bands_dev, w_dev, rows, taps,
                                                                                     nbands, taps_dev);
    DGC_LAUNCHED(ctx, "tap_map_tile");
    return DGC_OK;
  }
  if ((double)rows * nbands * taps >= (double)(1 << 24)) {
    // (65 bands: rows of 260 bytes are not 16-byte aligned; the matmul then fetches its operands with 4-byte
    // asynchronous copies instead of 16-byte ones, which is cheaper than a padding pass over the bands)
    return dgc_gemm_nt(ctx, bands_dev, w_dev, rows, taps, nbands, taps_dev);
  }
  size_t smem = ((((size_t)taps * (nbands | 1) + 3) & ~(size_t)3) + (size_t)nbands * 16) * sizeof(float);
  DGC_REQUIRE(ctx, smem <= 200 * 1024, "taps*nbands too large for shared memory");
  DGC_CUDA(ctx, cudaFuncSetAttribute(bands_to_taps_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  bands_to_taps_kernel<<<dgc_div_up(rows, 16 * BT_PASSES), 256, smem, ctx->stream>>>(bands_dev, w_dev, rows, nbands, taps,
                                                                          taps_dev);
  DGC_LAUNCHED(ctx, "bands_to_taps");
  return DGC_OK;
}
