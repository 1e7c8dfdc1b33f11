/*
 * CPU oracle for the frame-parallel render path -- TEST INFRASTRUCTURE, not product code.
 *
 * This header is a restatement, in plain scalar C, of what the reference's C backend
 * computes for each primitive on the path.  It is included twice by dgen_oracle.c:
 * once with R=float (the "C-backend-faithful" fp32 model: one rounding per operation in
 * the order the generated scalar loops perform them) and once with R=double (the fp64
 * evaluation used as the gradient reference).  Every function cites the reference file
 * and lines it follows (paths are relative to the reference project root).
 *
 * Layout convention of the oracle and of the CUDA kernels: batched audio is voice-major
 * `[B][T]` (the reference arena stores SignalTensors frame-major `[frame][elem]`,
 * Sources/DGenLazy/Realize.swift:418-436; the layout is a property of the boundary, the
 * arithmetic per (voice, frame) is identical).
 */

#ifndef ORC_CAT
#define ORC_CAT_(a, b) a##b
#define ORC_CAT(a, b) ORC_CAT_(a, b)
#endif
#define FN(name) ORC_CAT(name, SFX)

/* ---------------------------------------------------------------------------------------------
 * accum (scalar): Sources/DGen/Definitions.swift:215-246 (u_accum); the emitted C is visible in
 * toolchain/generated/hermetic/spectral-effect.c:89-106.  Output is the PRE-update state.
 *   next = acc + incr ; k = floor((next-min)/span) ; w = next - k*span ;
 *   state = w ; if (w >= max) state = w - span.
 * ------------------------------------------------------------------------------------------- */
void FN(orc_accum)(R incr, R mn, R mx, int T, R state0, R *out, R *state_out) {
  R acc = state0;
  const R span = mx - mn;
  for (int n = 0; n < T; ++n) {
    out[n] = acc;
    R next = acc + incr;
    R rel = next - mn;
    R k = FLOOR(rel / span);
    R w = next - k * span;
    acc = w;
    if (w >= mx) acc = w - span;
  }
  if (state_out) *state_out = acc;
}

/* ---------------------------------------------------------------------------------------------
 * Stateful tensor phasor: Sources/DGen/Emit+State.swift:322-369.
 *   incr = freq / sr ; next = prev + incr ; w = next - floor(next) ; if (w >= 1) w -= 1.
 * freq is [T][L] (time-varying per lane).  phase out [T][L] is the pre-update phase.
 * ------------------------------------------------------------------------------------------- */
void FN(orc_phasor_stateful)(const R *freq, int T, int L, R sr, R *phase) {
  for (int l = 0; l < L; ++l) {
    R prev = 0;
    for (int n = 0; n < T; ++n) {
      phase[(size_t)n * L + l] = prev;
      R incr = freq[(size_t)n * L + l] / sr;
      R next = prev + incr;
      R w = next - FLOOR(next);
      if (w >= (R)1) w = w - (R)1;
      prev = w;
    }
  }
}

/* deterministicPhasor: Sources/DGen/Emit+State.swift:370-387.
 *   phase[n] = frac((freq/sr) * n), stateless; used for Tensor-of-constant frequencies
 *   (Sources/DGenLazy/SignalTensor.swift:66-81). */
void FN(orc_phasor_deterministic)(const R *freq, int T, int L, R sr, R *phase) {
  for (int n = 0; n < T; ++n)
    for (int l = 0; l < L; ++l) {
      R inc = freq[l] / sr;
      R raw = inc * (R)n;
      phase[(size_t)n * L + l] = raw - FLOOR(raw);
    }
}

/* ---------------------------------------------------------------------------------------------
 * sampleRow / peekRow: Sources/DGen/Emit+RowSelection.swift:145-213.
 *   idx = fmod(i, R) (+R if negative); lo = floor; hi = lo+1 (wraps to row 0); lerp.
 * Returns lo, hi, frac for one playhead value.
 * ------------------------------------------------------------------------------------------- */
static inline void FN(orc_row_pos)(R idx, int rows, int *lo, int *hi, R *frac) {
  R w = FMOD(idx, (R)rows);
  if (w < 0) w = w + (R)rows;
  R fl = FLOOR(w);
  R ce = fl + (R)1;
  if (ce >= (R)rows) ce = 0;
  *lo = (int)fl;
  *hi = (int)ce;
  *frac = w - fl;
}

void FN(orc_sample_row)(const R *table, int rows, int cols, const R *idx, int T, R *out) {
  for (int n = 0; n < T; ++n) {
    int lo, hi;
    R fr;
    FN(orc_row_pos)(idx[n], rows, &lo, &hi, &fr);
    R omf = (R)1 - fr;
    for (int c = 0; c < cols; ++c)
      out[(size_t)n * cols + c] = omf * table[(size_t)lo * cols + c] + fr * table[(size_t)hi * cols + c];
  }
}

/* Control playhead of the batched harmonic synth: Examples/HarmonicE2E/Synth.swift:57-70.
 *   step = (F-1)/(T-1) in Float; playhead = clip(accum(step, min 0, max F-1), 0, F-1-1e-4). */
void FN(orc_playhead)(int F, int T, R *out) {
  R fmax = (R)(F > 1 ? F - 1 : 0);
  R denom = (R)(T > 1 ? T - 1 : 1);
  R step = fmax / denom;
  R hi = fmax - (R)1e-4f;
  if (hi < 0) hi = 0;
  if (fmax <= 0) {
    for (int n = 0; n < T; ++n) out[n] = 0;
    return;
  }
  FN(orc_accum)(step, 0, fmax, T, 0, out, 0);
  for (int n = 0; n < T; ++n) {
    R v = out[n];
    if (v < 0) v = 0;
    if (v > hi) v = hi;
    out[n] = v;
  }
}

/* ---------------------------------------------------------------------------------------------
 * Oscillator bank with constant per-partial frequency and amplitude (config "oscillator bank ->
 * filter -> FFT"):  audio[n] = sum_k sin(phase_k[n] * 2pi) * amp_k, summed k = 0..K-1 in order.
 * `2pi` is the Float constant 6.2831855 (toolchain/generated/hermetic/scalar-synth.c:66).
 * stateful != 0 selects the stateful phasor recurrence, else the deterministic phasor.
 * ------------------------------------------------------------------------------------------- */
void FN(orc_osc_bank_const)(const R *freq, const R *amp, int K, int T, R sr, int stateful, R *audio) {
  R *prev = (R *)calloc((size_t)K, sizeof(R));
  const R twopi = (R)TWO_PI_CONST;
  for (int n = 0; n < T; ++n) {
    R acc = 0;
    for (int k = 0; k < K; ++k) {
      R ph;
      R incr = freq[k] / sr;
      if (stateful) {
        ph = prev[k];
        R next = ph + incr;
        R w = next - FLOOR(next);
        if (w >= (R)1) w = w - (R)1;
        prev[k] = w;
      } else {
        R raw = incr * (R)n;
        ph = raw - FLOOR(raw);
      }
      acc = acc + SIN(ph * twopi) * amp[k];
    }
    audio[n] = acc;
  }
  free(prev);
}

/* ---------------------------------------------------------------------------------------------
 * history feedback one-pole  y[n] = x[n] + a*y[n-1]: historyRead/historyWrite semantics,
 * Sources/DGen/Emit+State.swift:150-224 (read-before-write gives the one-sample delay).
 * ------------------------------------------------------------------------------------------- */
void FN(orc_onepole)(const R *x, int T, R a, R y0, R *y) {
  R prev = y0;
  for (int n = 0; n < T; ++n) {
    R v = x[n] + a * prev;
    y[n] = v;
    prev = v;
  }
}

/* ---------------------------------------------------------------------------------------------
 * Graph.biquad, modes 0..5: Sources/DGen/HigherOps.swift:401-570 (the expression DAG is
 * restated node by node, same association order); selector is 1-based on mode+1
 * (Sources/DGen/Renderer/CRenderer.swift:953-979).  Coefficients are re-evaluated per frame in
 * the reference; with constant cutoff/Q/gain they are loop-invariant, so they are computed once.
 * ------------------------------------------------------------------------------------------- */
typedef struct { R b0, b1, b2, a1, a2; } FN(OrcBiquadCoef);

static R FN(orc_selector)(R mode1, const R *opt, int nopt) {
  if (mode1 <= 0) return 0;
  for (int i = 0; i < nopt; ++i)
    if (mode1 <= (R)(i + 1)) return opt[i];
  return 0;
}

void FN(orc_biquad_coef)(R cutoff, R q, R gain, R mode, FN(OrcBiquadCoef) *c) {
  R add4 = mode + (R)1;
  R mult7 = FABS(cutoff) * (R)0.00014247585730565955;
  R cos8 = COS(mult7);
  R mult9 = cos8 * (R)-1;
  R add10 = mult9 + (R)1;
  R div11 = add10 / (R)2;
  R sub12 = mult9 - (R)1;
  R div13 = sub12 / (R)-2;
  R sin14 = SIN(mult7);
  R mult15 = sin14 * (R)0.5;
  R abs17 = FABS(q);
  R div18 = mult15 / abs17;
  R mult19 = div18 * (R)-1;
  R mult20 = div18 * abs17;
  R mult21 = mult20 * (R)-1;
  R add22 = div18 + (R)1;
  R recip24 = (R)1 / add22;
  R mult26 = recip24 * gain;
  R mult31 = mult9 * (R)2;
  R not_sub35 = (R)1 - div18;
  /* shelf coefficients, modes 6 (high shelf) and 7 (low shelf): HigherOps.swift:468-528 */
  R A = SQRT(FABS(gain));
  R cosW0Pos = mult9 * (R)-1;
  R alphaShelf = sin14 / ((R)2.0 * abs17);
  R Ap1 = A + (R)1, Am1 = A - (R)1;
  R Ap1_cos = Ap1 * cosW0Pos, Am1_cos = Am1 * cosW0Pos;
  R twoSqrtA_alpha = ((R)2.0 * SQRT(A)) * alphaShelf;
  R hs_b0 = A * ((Ap1 + Am1_cos) + twoSqrtA_alpha);
  R hs_b1 = (R)-2.0 * (A * (Am1 + Ap1_cos));
  R hs_b2 = A * ((Ap1 + Am1_cos) - twoSqrtA_alpha);
  R hs_a0 = (Ap1 - Am1_cos) + twoSqrtA_alpha;
  R ls_b0 = A * ((Ap1 - Am1_cos) + twoSqrtA_alpha);
  R ls_b1 = (R)2.0 * (A * (Am1 - Ap1_cos));
  R ls_b2 = A * ((Ap1 - Am1_cos) - twoSqrtA_alpha);
  R ls_a0 = (Ap1 + Am1_cos) + twoSqrtA_alpha;
  R hs_a1n = ((R)2.0 * (Am1 - Ap1_cos)) / hs_a0, hs_a2n = ((Ap1 - Am1_cos) - twoSqrtA_alpha) / hs_a0;
  R ls_a1n = ((R)-2.0 * (Am1 + Ap1_cos)) / ls_a0, ls_a2n = ((Ap1 + Am1_cos) - twoSqrtA_alpha) / ls_a0;
  R o23[8] = {div11, div13, mult19, mult21, (R)1, add22, hs_b2 / hs_a0, ls_b2 / ls_a0};
  R o32[8] = {add10, sub12, 0, 0, mult31, mult31, hs_b1 / hs_a0, ls_b1 / ls_a0};
  R o36[8] = {div11, div13, div18, mult20, (R)1, not_sub35, hs_b0 / hs_a0, ls_b0 / ls_a0};
  /* modes 0-5 scale by gain / a0; the shelves carry the gain in A (isShelfMode = mode >= 6, :533-548) */
  int shelf = mode >= (R)6;
  R s23 = FN(orc_selector)(add4, o23, 8), s32 = FN(orc_selector)(add4, o32, 8), s36 = FN(orc_selector)(add4, o36, 8);
  c->b2 = shelf ? s23 : s23 * mult26;
  c->b1 = shelf ? s32 : s32 * mult26;
  c->b0 = shelf ? s36 : s36 * mult26;
  c->a2 = shelf ? (mode >= (R)7 ? ls_a2n : hs_a2n) : not_sub35 * recip24;
  c->a1 = shelf ? (mode >= (R)7 ? ls_a1n : hs_a1n) : mult31 * recip24;
}

/* y = ((b2*x2 + b1*x1) + b0*x0) - (a2*y2 + a1*y1)   (HigherOps.swift:532-567) */
void FN(orc_biquad)(const R *x, int T, R cutoff, R q, R gain, R mode, R *y) {
  FN(OrcBiquadCoef) c;
  FN(orc_biquad_coef)(cutoff, q, gain, mode, &c);
  R x1 = 0, x2 = 0, y1 = 0, y2 = 0;
  for (int n = 0; n < T; ++n) {
    R x0 = x[n];
    R add39 = (x2 * c.b2 + x1 * c.b1) + x0 * c.b0;
    R add45 = y2 * c.a2 + y1 * c.a1;
    R v = add39 - add45;
    y[n] = v;
    x2 = x1; x1 = x0; y2 = y1; y1 = v;
  }
}

/* The same recurrence with GIVEN coefficients (b0 b1 b2 a1 a2).  In double with the single-precision
 * coefficients it is the exact response of the filter the fp32 graph defines: the yardstick for how much of a
 * difference between two fp32 evaluations is rounding noise of the recurrence itself. */
void FN(orc_biquad_with_coef)(const R *x, int T, const R *coef, R *y) {
  R x1 = 0, x2 = 0, y1 = 0, y2 = 0;
  for (int n = 0; n < T; ++n) {
    R x0 = x[n];
    R v = ((x2 * coef[2] + x1 * coef[1]) + x0 * coef[0]) - (y2 * coef[4] + y1 * coef[3]);
    y[n] = v;
    x2 = x1; x1 = x0; y2 = y1; y1 = v;
  }
}

/* Tensor biquad bank: x [B][T] shared by L lanes, y [B][L][T].  Lane independence is exact
 * (Tests/DGenLazyTests/TensorBiquadGradientTests.swift). */
void FN(orc_biquad_bank)(const R *x, int B, int T, int L, const R *cutoff, const R *q, R gain, R mode, R *y) {
  for (int b = 0; b < B; ++b)
    for (int l = 0; l < L; ++l)
      FN(orc_biquad)(x + (size_t)b * T, T, cutoff[l], q[l], gain, mode, y + ((size_t)b * L + l) * T);
}

/* ---------------------------------------------------------------------------------------------
 * Gradient reference for the biquad bank: loss = scale * sum_{b,l,n} (y - target)^2, gradients
 * w.r.t. per-lane cutoff and q through the recurrence (what BPTT computes,
 * Sources/DGen/Gradients.swift:765-778): adjoint lam[n] = g[n] - a1 lam[n+1] - a2 lam[n+2],
 * dL/db_i = sum lam[n] x[n-i], dL/da_i = -sum lam[n] y[n-i]; the coefficient Jacobian is taken by
 * central differences of orc_biquad_coef in this precision (meant for R = double).
 * x [B][T], target [B][L][T] (oracle layout).  Returns the loss.
 * ------------------------------------------------------------------------------------------- */
double FN(orc_biquad_bank_mse_grad)(const R *x, int B, int T, int L, const R *cutoff, const R *q, R gain, R mode,
                                    const R *target, R scale, R *gcut, R *gq) {
  R *y = (R *)malloc(sizeof(R) * T), *lam = (R *)malloc(sizeof(R) * (T + 2));
  double loss = 0;
  for (int l = 0; l < L; ++l) {
    FN(OrcBiquadCoef) c;
    FN(orc_biquad_coef)(cutoff[l], q[l], gain, mode, &c);
    double G[5] = {0, 0, 0, 0, 0};
    for (int b = 0; b < B; ++b) {
      const R *xb = x + (size_t)b * T, *tb = target + ((size_t)b * L + l) * T;
      FN(orc_biquad)(xb, T, cutoff[l], q[l], gain, mode, y);
      lam[T] = 0; lam[T + 1] = 0;
      for (int n = T - 1; n >= 0; --n) {
        R d = y[n] - tb[n];
        loss += (double)scale * (double)d * (double)d;
        lam[n] = (R)2 * scale * d - c.a1 * lam[n + 1] - c.a2 * lam[n + 2];
        G[0] += (double)lam[n] * (double)xb[n];
        if (n >= 1) { G[1] += (double)lam[n] * (double)xb[n - 1]; G[3] -= (double)lam[n] * (double)y[n - 1]; }
        if (n >= 2) { G[2] += (double)lam[n] * (double)xb[n - 2]; G[4] -= (double)lam[n] * (double)y[n - 2]; }
      }
    }
    R hc = FABS(cutoff[l]) * (R)1e-5 + (R)1e-7, hq = FABS(q[l]) * (R)1e-5 + (R)1e-7;
    FN(OrcBiquadCoef) cp, cm, qp, qm;
    FN(orc_biquad_coef)(cutoff[l] + hc, q[l], gain, mode, &cp);
    FN(orc_biquad_coef)(cutoff[l] - hc, q[l], gain, mode, &cm);
    FN(orc_biquad_coef)(cutoff[l], q[l] + hq, gain, mode, &qp);
    FN(orc_biquad_coef)(cutoff[l], q[l] - hq, gain, mode, &qm);
    const R *pp = (const R *)&cp, *pm = (const R *)&cm, *rp = (const R *)&qp, *rm = (const R *)&qm;
    double dc = 0, dq = 0;
    for (int i = 0; i < 5; ++i) {
      dc += G[i] * ((double)pp[i] - (double)pm[i]) / (2.0 * (double)hc);
      dq += G[i] * ((double)rp[i] - (double)rm[i]) / (2.0 * (double)hq);
    }
    gcut[l] = (R)dc;
    gq[l] = (R)dq;
  }
  free(y); free(lam);
  return loss;
}

/* ---------------------------------------------------------------------------------------------
 * Host FFT service: Sources/DGenHostSupport/DGenHostSupport.c:10-30 wraps vDSP_fft_zip (Apple
 * Accelerate, closed source, version = whatever the OS ships).  Its published definition is the
 * unnormalised complex DFT  X[k] = sum x[n] exp(-+2 pi i k n / N)  on split re/im arrays, in
 * place, both directions unscaled.  Restated as an iterative radix-2 decimation-in-time FFT with
 * twiddles evaluated in double and rounded to R.
 * ------------------------------------------------------------------------------------------- */
void FN(orc_fft)(R *re, R *im, int N, int inverse) {
  int j = 0;
  for (int i = 1; i < N; ++i) {
    int bit = N >> 1;
    for (; j & bit; bit >>= 1) j ^= bit;
    j ^= bit;
    if (i < j) {
      R t = re[i]; re[i] = re[j]; re[j] = t;
      t = im[i]; im[i] = im[j]; im[j] = t;
    }
  }
  for (int len = 2; len <= N; len <<= 1) {
    int half = len >> 1;
    for (int k = 0; k < half; ++k) {
      double ang = 2.0 * M_PI * (double)k / (double)len;
      R wr = (R)cos(ang);
      R wi = (R)(inverse ? sin(ang) : -sin(ang));
      for (int i = k; i < N; i += len) {
        int jj = i + half;
        R tr = wr * re[jj] - wi * im[jj];
        R ti = wr * im[jj] + wi * re[jj];
        re[jj] = re[i] - tr; im[jj] = im[i] - ti;
        re[i] = re[i] + tr;  im[i] = im[i] + ti;
      }
    }
  }
}

/* hann(n), periodic: Sources/DGenLazy/SpectralTensorOps.swift:42-49 (Float arithmetic). */
void FN(orc_hann_periodic)(int N, R *w) {
  R scale = (R)2 * (R)PI_CONST / (R)N;
  for (int i = 0; i < N; ++i) w[i] = (R)0.5 - (R)0.5 * COS(scale * (R)i);
}

/* Symmetric Hann of the spectral loss: Sources/DGen/HigherOps.swift:72-76 (Double, then Float). */
void FN(orc_hann_symmetric)(int N, R *w) {
  for (int i = 0; i < N; ++i)
    w[i] = (R)(float)(0.5 * (1.0 - cos(2.0 * M_PI * (double)i / (double)(N - 1))));
}

/* ---------------------------------------------------------------------------------------------
 * buffer(size:N, hop:) -> FFT -> magnitude.
 * bufferView: Sources/DGen/HigherOps.swift:738-792; window element i at frame f = x[f-N+1+i],
 * zero before the start; downstream blocks run at frames f = 0, hop, 2hop, ...
 * acceleratedFFT: Sources/DGen/Emit+AcceleratedFFT.swift:16-112 (real input, imaginary = 0, full
 * complex transform).  mags is [H][N/2+1], H = ceil(T/hop).  window may be NULL (rectangular).
 * ------------------------------------------------------------------------------------------- */
void FN(orc_buffer_fft_mag)(const R *x, int T, int N, int hop, const R *window, R *mags) {
  R *re = (R *)malloc(sizeof(R) * N), *im = (R *)malloc(sizeof(R) * N);
  int nb = N / 2 + 1, h = 0;
  for (int f = 0; f < T; f += hop, ++h) {
    for (int i = 0; i < N; ++i) {
      int t = f - N + 1 + i;
      R v = t >= 0 ? x[t] : 0;
      re[i] = window ? v * window[i] : v;
      im[i] = 0;
    }
    FN(orc_fft)(re, im, N, 0);
    for (int k = 0; k < nb; ++k) mags[(size_t)h * nb + k] = SQRT(re[k] * re[k] + im[k] * im[k]);
  }
  free(re); free(im);
}

/* ---------------------------------------------------------------------------------------------
 * overlapAdd: Sources/DGen/Emit+FFT.swift:6-62.  The ring is followed literally so that the
 * order in which overlapping windows are added matches.  frames [H][N] are the windows scattered
 * at hop frames 0, hop, ...
 * ------------------------------------------------------------------------------------------- */
void FN(orc_overlap_add)(const R *frames, int T, int N, int hop, R *out) {
  R *ring = (R *)calloc((size_t)N, sizeof(R));
  int readPos = 0, counter = 0, h = 0;
  for (int t = 0; t < T; ++t) {
    if (counter == 0) {
      for (int i = 0; i < N; ++i) {
        int p = readPos + i;
        if (p >= N) p -= N;
        ring[p] = ring[p] + frames[(size_t)h * N + i];
      }
      ++h;
    }
    out[t] = ring[readPos];
    ring[readPos] = 0;
    if (++readPos >= N) readPos = 0;
    if (++counter >= hop) counter = 0;
  }
  free(ring);
}

/* ---------------------------------------------------------------------------------------------
 * partitionedConvolve: Sources/DGenLazy/SpectralTensorOps.swift:204-254;
 * MAC ring: Sources/DGen/Emit+PartitionedConvolution.swift:26-113 and
 * Sources/DGen/Renderer/CRenderer.swift:1243-1274 (K calls of complex multiply-accumulate, k = 0
 * first); IFFT scaled by 1/N: Sources/DGen/Emit+AcceleratedFFT.swift:92-107.
 *   X_h = FFT(hann ⊙ window_h) ; H_k = FFT(zero-pad(ir[k*hop:(k+1)*hop], N)) ;
 *   Y_h = sum_{k<K} X_{h-k} * H_k ; out = overlapAdd(IFFT(Y_h)/N * hann * gain, hop).
 * ------------------------------------------------------------------------------------------- */
void FN(orc_partitioned_convolve)(const R *x, int T, const R *ir, int irlen, int N, int hop, R gain, R *out) {
  int K = (irlen + hop - 1) / hop;
  if (K < 1) K = 1;
  int H = (T + hop - 1) / hop;
  R *win = (R *)malloc(sizeof(R) * N);
  FN(orc_hann_periodic)(N, win);
  R *hre = (R *)calloc((size_t)K * N, sizeof(R)), *him = (R *)calloc((size_t)K * N, sizeof(R));
  for (int k = 0; k < K; ++k) {
    for (int i = 0; i < hop && k * hop + i < irlen; ++i) hre[(size_t)k * N + i] = ir[k * hop + i];
    FN(orc_fft)(hre + (size_t)k * N, him + (size_t)k * N, N, 0);
  }
  R *xre = (R *)calloc((size_t)H * N, sizeof(R)), *xim = (R *)calloc((size_t)H * N, sizeof(R));
  R *frames = (R *)malloc(sizeof(R) * (size_t)H * N);
  R *yre = (R *)malloc(sizeof(R) * N), *yim = (R *)malloc(sizeof(R) * N);
  for (int h = 0; h < H; ++h) {
    int f = h * hop;
    R *re = xre + (size_t)h * N, *im = xim + (size_t)h * N;
    for (int i = 0; i < N; ++i) {
      int t = f - N + 1 + i;
      re[i] = (t >= 0 ? x[t] : 0) * win[i];
      im[i] = 0;
    }
    FN(orc_fft)(re, im, N, 0);
    for (int i = 0; i < N; ++i) { yre[i] = 0; yim[i] = 0; }
    for (int k = 0; k < K && k <= h; ++k) {
      const R *ar = xre + (size_t)(h - k) * N, *ai = xim + (size_t)(h - k) * N;
      const R *br = hre + (size_t)k * N, *bi = him + (size_t)k * N;
      for (int i = 0; i < N; ++i) {
        yre[i] = yre[i] + (ar[i] * br[i] - ai[i] * bi[i]);
        yim[i] = yim[i] + (ar[i] * bi[i] + ai[i] * br[i]);
      }
    }
    FN(orc_fft)(yre, yim, N, 1);
    R invn = (R)1 / (R)N;
    for (int i = 0; i < N; ++i) frames[(size_t)h * N + i] = ((yre[i] * invn) * win[i]) * gain;
  }
  FN(orc_overlap_add)(frames, T, N, hop, out);
  free(win); free(hre); free(him); free(xre); free(xim); free(frames); free(yre); free(yim);
}

/* ---------------------------------------------------------------------------------------------
 * spectralLossFFTBatched forward: Sources/DGen/HigherOps.swift:165-263 (tables) and
 * Sources/DGen/Emit+SpectralLoss.swift:719-938 (per (hop frame, batch) body + batch mean).
 *   window at hop frame f:  s[n] = x[f-(N-1)+n] * hannS[n]   (0 outside [0,T))
 *   radix-2 DIT with the reference's twiddle table (cos, sin in Double rounded to Float, negated
 *   imaginary for the forward transform), butterflies in the reference's order;
 *   m[k] = sqrt(re^2+im^2), k = 0..N/2 ;  d = use_log ? log(m1+eps)-log(m2+eps) : m1-m2 ;
 *   partial[h][b] = sum_k |d|  (L1)  or  sum_k d^2 (L2).
 * x1, x2 are [B][T].  partial is [H][B] with H = ceil(T/hop) (the reference's scratchCell
 * layout).  Returns sum over hop frames of (sum_b partial)/B, accumulated in double.
 * eps = 1e-8 (Sources/DGen/GradientConfig.swift:38).
 * ------------------------------------------------------------------------------------------- */
static void FN(orc_loss_fft)(R *re, R *im, int N, const R *twre, const R *twim) {
  int stages = 0;
  while ((1 << stages) < N) ++stages;
  for (int i = 0; i < N; ++i) {
    int rev = 0, bits = i;
    for (int s = 0; s < stages; ++s) { rev = rev * 2 + (bits & 1); bits >>= 1; }
    if (i < rev) {
      R t = re[i]; re[i] = re[rev]; re[rev] = t;
      t = im[i]; im[i] = im[rev]; im[rev] = t;
    }
  }
  for (int s = 0; s < stages; ++s) {
    int bsize = 1 << (s + 1), half = bsize >> 1, nb = (N / bsize) * half;
    for (int flat = 0; flat < nb; ++flat) {
      int group = flat / half, k = flat - group * half;
      int i = group * bsize + k, j = i + half;
      R wr = twre[half - 1 + k], wi = (R)0 - twim[half - 1 + k];
      R tr = wr * re[j] - wi * im[j];
      R ti = wr * im[j] + wi * re[j];
      R ar = re[i], ai = im[i];
      re[i] = ar + tr; im[i] = ai + ti;
      re[j] = ar - tr; im[j] = ai - ti;
    }
  }
}

double FN(orc_spectral_loss)(const R *x1, const R *x2, int B, int T, int N, int hop, int use_log,
                             int l2, R *partial) {
  int nb = N / 2 + 1, stages = 0;
  while ((1 << stages) < N) ++stages;
  R *win = (R *)malloc(sizeof(R) * N);
  FN(orc_hann_symmetric)(N, win);
  R *twre = (R *)malloc(sizeof(R) * N), *twim = (R *)malloc(sizeof(R) * N);
  for (int s = 0; s < stages; ++s) {
    int half = 1 << s;
    for (int k = 0; k < half; ++k) {
      double ang = 2.0 * M_PI * (double)k / (double)(2 * half);
      twre[half - 1 + k] = (R)(float)cos(ang);
      twim[half - 1 + k] = (R)(float)sin(ang);
    }
  }
  R *re = (R *)malloc(sizeof(R) * N), *im = (R *)malloc(sizeof(R) * N);
  R *m1 = (R *)malloc(sizeof(R) * nb), *m2 = (R *)malloc(sizeof(R) * nb);
  const R eps = (R)1e-8f;
  double total = 0;
  int h = 0;
  for (int f = 0; f < T; f += hop, ++h) {
    R frame = 0;
    for (int b = 0; b < B; ++b) {
      for (int sig = 0; sig < 2; ++sig) {
        const R *x = (sig ? x2 : x1) + (size_t)b * T;
        R *m = sig ? m2 : m1;
        for (int n = 0; n < N; ++n) {
          int t = f - (N - 1) + n;
          R s = (t >= 0 && t < T) ? x[t] : 0;
          re[n] = s * win[n];
          im[n] = 0;
        }
        FN(orc_loss_fft)(re, im, N, twre, twim);
        for (int k = 0; k < nb; ++k) m[k] = SQRT(re[k] * re[k] + im[k] * im[k]);
      }
      R acc = 0;
      for (int k = 0; k < nb; ++k) {
        R d = use_log ? (LOG(m1[k] + eps) - LOG(m2[k] + eps)) : (m1[k] - m2[k]);
        acc = acc + (l2 ? d * d : FABS(d));
      }
      if (partial) partial[(size_t)h * B + b] = acc;
      frame = frame + acc;
    }
    total += (double)(frame / (R)B);
  }
  free(win); free(twre); free(twim); free(re); free(im); free(m1); free(m2);
  return total;
}

/* Multi-scale loss in the HarmonicE2E style: Examples/HarmonicE2E/Trainer.swift:538-588.
 * For each window size: L1 linear-magnitude loss and L1 log-magnitude loss, hop = N/hop_div,
 * normalize:true divides each by the frame count (Sources/DGenLazy/Functions.swift:951-954);
 * lin terms weighted w_lin/nscales, log terms w_log/nscales.  Returns sum over frames. */
double FN(orc_mss_loss)(const R *x1, const R *x2, int B, int T, const int *sizes, int nscales, int hop_div,
                        R w_lin, R w_log) {
  double total = 0;
  int usable = 0;
  for (int s = 0; s < nscales; ++s)
    if (sizes[s] > 1 && sizes[s] <= T) ++usable;
  for (int s = 0; s < nscales; ++s) {
    int N = sizes[s];
    if (N <= 1 || N > T) continue;
    int hop = N / (hop_div > 0 ? hop_div : 1);
    if (hop < 1) hop = 1;
    double lin = w_lin != 0 ? FN(orc_spectral_loss)(x1, x2, B, T, N, hop, 0, 0, 0) : 0;
    double lg = w_log != 0 ? FN(orc_spectral_loss)(x1, x2, B, T, N, hop, 1, 0, 0) : 0;
    total += (lin * (double)w_lin + lg * (double)w_log) / (double)usable / (double)T;
  }
  return total;
}

/* ---------------------------------------------------------------------------------------------
 * Gradient of orc_mss_loss w.r.t. x1 (the prediction), following the reference's backward rules
 * (Sources/DGen/Emit+SpectralLoss.swift:940-1325, Sources/DGen/Gradients.swift:1038-1142):
 *   gradMag1 = sign(d)            (linear term)   or  sign(dlog) / (m1 + eps)   (log term), times c;
 *   gradX1[k] = gradMag1 * X1[k] / max(m1, 1e-8), k = 0..N/2, zero above;
 *   time gradient = Re(unnormalised inverse transform of gradX1) * hann; summed over covering windows.
 * c = upstream * w / (B * usable * T).  grad [B][T] is overwritten.  Meant for R = double.
 * ------------------------------------------------------------------------------------------- */
void FN(orc_mss_loss_grad)(const R *x1, const R *x2, int B, int T, const int *sizes, int nscales, int hop_div,
                           R w_lin, R w_log, R upstream, R *grad) {
  int usable = 0;
  for (int s = 0; s < nscales; ++s)
    if (sizes[s] > 1 && sizes[s] <= T) ++usable;
  for (size_t i = 0; i < (size_t)B * T; ++i) grad[i] = 0;
  const R eps = (R)1e-8f;
  for (int s = 0; s < nscales; ++s) {
    int N = sizes[s];
    if (N <= 1 || N > T) continue;
    int hop = N / (hop_div > 0 ? hop_div : 1);
    if (hop < 1) hop = 1;
    R c_lin = upstream * w_lin / ((R)B * (R)usable * (R)T), c_log = upstream * w_log / ((R)B * (R)usable * (R)T);
    R *win = (R *)malloc(sizeof(R) * N);
    FN(orc_hann_symmetric)(N, win);
    R *r1 = (R *)malloc(sizeof(R) * N), *i1 = (R *)malloc(sizeof(R) * N);
    R *r2 = (R *)malloc(sizeof(R) * N), *i2 = (R *)malloc(sizeof(R) * N);
    for (int b = 0; b < B; ++b)
      for (int f = 0; f < T; f += hop) {
        for (int n = 0; n < N; ++n) {
          int t = f - (N - 1) + n;
          int ok = t >= 0 && t < T;
          r1[n] = ok ? x1[(size_t)b * T + t] * win[n] : 0; i1[n] = 0;
          r2[n] = ok ? x2[(size_t)b * T + t] * win[n] : 0; i2[n] = 0;
        }
        FN(orc_fft)(r1, i1, N, 0);
        FN(orc_fft)(r2, i2, N, 0);
        for (int k = 0; k < N; ++k) {
          if (k > N / 2) { r1[k] = 0; i1[k] = 0; continue; }
          R m1 = SQRT(r1[k] * r1[k] + i1[k] * i1[k]), m2 = SQRT(r2[k] * r2[k] + i2[k] * i2[k]);
          R d = m1 - m2, dl = LOG(m1 + eps) - LOG(m2 + eps);
          R sd = d > 0 ? (R)1 : (d < 0 ? (R)-1 : 0), sl = dl > 0 ? (R)1 : (dl < 0 ? (R)-1 : 0);
          R gm = c_lin * sd + c_log * sl / (m1 + eps);
          R safe = m1 > (R)1e-8f ? m1 : (R)1e-8f;
          r1[k] = gm * r1[k] / safe;
          i1[k] = gm * i1[k] / safe;
        }
        FN(orc_fft)(r1, i1, N, 1);
        for (int n = 0; n < N; ++n) {
          int t = f - (N - 1) + n;
          if (t >= 0 && t < T) grad[(size_t)b * T + t] += r1[n] * win[n];
        }
      }
    free(win); free(r1); free(i1); free(r2); free(i2);
  }
}

/* ---------------------------------------------------------------------------------------------
 * Batched harmonic + FIR-noise synthesis: Examples/HarmonicE2E/Synth.swift:47-102.
 *   playhead -> sampleRow of f0/uv [F][B], amps [F][B][K], gain/noise_gain [F][B],
 *   taps [F][B][FIR]; Nyquist mask + renormalise (Synth.swift:161-170); stateful phasor of
 *   k*f0 (Emit+State.swift:322-369); sin(phase*2pi); sum over partials * gain * uv * hscale;
 *   noise: window w[i] = noise[n-FIR+1+i] (bufferView, HigherOps.swift:738-792),
 *   filtered = sum_i w[i]*taps[i]; out = harm + filtered * noise_gain * 0.12 * nscale.
 * noise is [B][T] (the configs supply per-voice noise; the reference shares one stream).
 * audio out [B][T].  phase_out (optional) [B][K][T] receives the pre-update phases.
 * ------------------------------------------------------------------------------------------- */
void FN(orc_harmonic_noise_render)(int B, int T, int K, int F, int FIR, R sr, const R *f0, const R *uv,
                                   const R *amps, const R *gain, const R *noise_gain, const R *taps,
                                   const R *noise, R hscale, R nscale, R *audio, R *phase_out) {
  R *play = (R *)malloc(sizeof(R) * T);
  FN(orc_playhead)(F, T, play);
  const R twopi = (R)TWO_PI_CONST;
  const R nyq = sr * (R)0.5;
  R *ph = (R *)malloc(sizeof(R) * K), *masked = (R *)malloc(sizeof(R) * K);
  for (int b = 0; b < B; ++b) {
    for (int k = 0; k < K; ++k) ph[k] = 0;
    for (int n = 0; n < T; ++n) {
      int lo, hi;
      R fr;
      FN(orc_row_pos)(play[n], F, &lo, &hi, &fr);
      R omf = (R)1 - fr;
#define LERP2(tab) (omf * (tab)[(size_t)lo * B + b] + fr * (tab)[(size_t)hi * B + b])
      R f0t = LERP2(f0), uvt = LERP2(uv), gt = LERP2(gain), ngt = LERP2(noise_gain);
#undef LERP2
      const R *alo = amps + ((size_t)lo * B + b) * K, *ahi = amps + ((size_t)hi * B + b) * K;
      R denom = 0;
      for (int k = 0; k < K; ++k) {
        R freq = (R)(k + 1) * f0t;
        R a = omf * alo[k] + fr * ahi[k];
        masked[k] = a * (freq < nyq ? (R)1 : (R)0);
        denom = denom + masked[k];
      }
      denom = denom + (R)1e-8f;
      R hsum = 0;
      for (int k = 0; k < K; ++k) {
        R freq = (R)(k + 1) * f0t;
        R p = ph[k];
        if (phase_out) phase_out[((size_t)b * K + k) * T + n] = p;
        R incr = freq / sr;
        R next = p + incr;
        R w = next - FLOOR(next);
        if (w >= (R)1) w = w - (R)1;
        ph[k] = w;
        hsum = hsum + SIN(p * twopi) * (masked[k] / denom);
      }
      R harm = ((hsum * gt) * uvt) * hscale;
      R nout = 0;
      if (FIR > 0) {
        const R *tlo = taps + ((size_t)lo * B + b) * FIR, *thi = taps + ((size_t)hi * B + b) * FIR;
        const R *xn = noise + (size_t)b * T;
        R acc = 0;
        for (int i = 0; i < FIR; ++i) {
          int t = n - FIR + 1 + i;
          R xv = t >= 0 ? xn[t] : 0;
          acc = acc + xv * (omf * tlo[i] + fr * thi[i]);
        }
        nout = ((acc * ngt) * (R)0.12f) * nscale;
      }
      audio[(size_t)b * T + n] = harm + nout;
    }
  }
  free(play); free(ph); free(masked);
}

/* ---------------------------------------------------------------------------------------------
 * Adam: Sources/DGenLazy/Optimizers.swift:164-243 (bias-corrected, eps outside the sqrt).
 * ------------------------------------------------------------------------------------------- */
void FN(orc_adam)(R *theta, const R *g, R *m, R *v, size_t n, int t, R lr, R b1, R b2, R eps) {
  R c1 = (R)1 - POW(b1, (R)t), c2 = (R)1 - POW(b2, (R)t);
  for (size_t i = 0; i < n; ++i) {
    m[i] = b1 * m[i] + ((R)1 - b1) * g[i];
    v[i] = b2 * v[i] + ((R)1 - b2) * g[i] * g[i];
    R mh = m[i] / c1, vh = v[i] / c2;
    theta[i] = theta[i] - lr * mh / (SQRT(vh) + eps);
  }
}

#undef FN
