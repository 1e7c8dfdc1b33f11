/*
 * dgen_cuda.h -- C ABI of libdgen_cuda.so: the sm_100a implementation of DGen's frame-parallel
 * render path (oscillator bank, linear recurrences, hop-gated FFT / overlap-add / partitioned
 * convolution, multi-scale spectral loss, controller matmul, Adam).
 *
 * This is the boundary a host (DGen's Swift `CUDALazyRuntime`, or any C caller) binds.  Plain
 * pointers and sizes only.  Every function returns a status (DGC_OK = 0, negative = error) and
 * never throws or aborts; dgc_last_error() gives the text for the last failure on a context.
 * All work is enqueued on the context's CUDA stream; dgc_sync() is the only blocking call.
 * One context per GPU; calls on one context must be serialised by the caller (the reference's
 * runtimes have the same rule: one global graph, not thread-safe, Sources/DGenLazy/LazyGraph.swift:241-264).
 *
 * Pointers named *_dev are CUDA device pointers (for example dgc_arena_ptr() + an offset, which
 * replaces the reference's host-visible `float *memory` arena, Sources/DGen/Runtime.swift:732-744);
 * pointers named *_host are ordinary host memory.
 *
 * Layouts.  Batched audio is voice-major `[B][T]` floats.  Control tables are `[F][B]` and
 * `[F][B][K]` exactly as Examples/HarmonicE2E/Synth.swift:72-75 builds them.  Lane signals of the
 * biquad bank are `[B][T][L]` (lanes fastest, the reference's frame-major tensor layout,
 * Sources/DGenLazy/Realize.swift:418-436).
 *
 * In the comments below "replaces" names the reference code whose work the entry point does.
 */
#ifndef DGEN_CUDA_H
#define DGEN_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DGC_ABI_VERSION 1

enum {
  DGC_OK = 0,
  DGC_ERR_INVALID = -1,   /* bad argument (null pointer, size out of range, unsupported shape) */
  DGC_ERR_CUDA = -2,      /* a CUDA runtime call or launch failed; text in dgc_last_error */
  DGC_ERR_OOM = -3,       /* device allocation failed */
  DGC_ERR_TIMEOUT = -4,   /* dgc_sync: the stream did not drain in time */
  DGC_ERR_DEVICE = -5,    /* a kernel reported a device-side error through the status word */
  DGC_ERR_UNSUPPORTED = -6
};

typedef struct dgc_ctx dgc_ctx;
typedef struct dgc_arena dgc_arena;

/* ---- context ------------------------------------------------------------------------------------
 * replaces: MetalCompiledKernel.init / CCompiledKernel.compileAndLoad as the owner of device,
 * queue and scratch (Sources/DGen/MetalRuntime.swift:40, Sources/DGen/Runtime.swift:240-340). */
int32_t dgc_abi_version(void);
int32_t dgc_ctx_create(int32_t device, dgc_ctx **out);
int32_t dgc_ctx_destroy(dgc_ctx *ctx);
const char *dgc_last_error(dgc_ctx *ctx);
/* external != 0: enqueue on the caller's CUDA stream (a cudaStream_t; NULL is CUDA's default stream).
 * external == 0: go back to the context's own stream. */
int32_t dgc_ctx_set_stream(dgc_ctx *ctx, void *cuda_stream, int32_t external);
/* Waits for the stream, at most timeout_ms (0 = no limit), then checks the device status word. */
int32_t dgc_sync(dgc_ctx *ctx, uint32_t timeout_ms);
/* Self-test of the failure reporting, without a fault and without an unbounded wait.
 * dgc_selftest_expired_wait enqueues a kernel that waits on a barrier nothing arrives on, with the bounded wait every
 * pipeline kernel of the library uses cut down to `polls` polls (1 .. 2^20): the wait gives up, the kernel writes
 * the status word and returns, and the next dgc_sync reports DGC_ERR_DEVICE (and clears the word).
 * dgc_selftest_busy keeps the stream busy for `milliseconds` (1 .. 500) so that a dgc_sync with a shorter timeout
 * returns DGC_ERR_TIMEOUT; the stream drains by itself and later calls work.  No reference counterpart. */
int32_t dgc_selftest_expired_wait(dgc_ctx *ctx, uint32_t polls);
int32_t dgc_selftest_busy(dgc_ctx *ctx, uint32_t milliseconds);
/* Event timing on the context's stream (replaces profileKernels, Sources/DGen/MetalRuntime.swift:397-425). */
int32_t dgc_profile_begin(dgc_ctx *ctx);
int32_t dgc_profile_end(dgc_ctx *ctx, float *elapsed_ms);
/* Number of kernels this library has launched on the context since creation. */
int64_t dgc_launch_count(dgc_ctx *ctx);

/* ---- arena --------------------------------------------------------------------------------------
 * replaces: the caller-owned flat float arena `state` of dgen_process_v1
 * (toolchain/include/dgen_runtime.h:282-288) and LazyRuntime.memoryPointer()
 * (Sources/DGenLazy/Realize.swift:12-19): device memory plus explicit upload / download. */
int32_t dgc_arena_create(dgc_ctx *ctx, uint64_t nfloats, dgc_arena **out);
/* An arena over device memory the CALLER owns (256-byte aligned; it stays the caller's: dgc_arena_destroy only drops
 * the handle): for hosts that allocate device memory themselves and want plans to address it. */
int32_t dgc_arena_wrap(dgc_ctx *ctx, float *dev, uint64_t nfloats, dgc_arena **out);
int32_t dgc_arena_destroy(dgc_arena *a);
float *dgc_arena_ptr(dgc_arena *a);
uint64_t dgc_arena_size(dgc_arena *a);
int32_t dgc_arena_zero(dgc_arena *a);                                          /* zeroAllBuffers */
int32_t dgc_arena_upload(dgc_arena *a, uint64_t offset, const float *src_host, uint64_t n);   /* injectTensorData */
int32_t dgc_arena_download(dgc_arena *a, uint64_t offset, float *dst_host, uint64_t n);       /* readOutputs / readGradients */

/* Builds the tables the context caches per (control frames F, frames T) -- the control playhead, the per-frame
 * control-row positions and the per-row frame ranges -- on the context stream and waits for them.  Every entry
 * point builds what it needs on first use; a host calls this up front when the first use must not allocate
 * or synchronise (real-time start-up), or before it drives one context from two streams.
 * No reference counterpart (the reference recomputes the clock inside every kernel). */
int32_t dgc_ctx_prepare_tables(dgc_ctx *ctx, int32_t F, int32_t T);

/* ---- scalar clocks ------------------------------------------------------------------------------
 * replaces: scalar `accum` (Sources/DGen/Definitions.swift:215-246): out[n] = state before the
 * n-th update, sequential single-precision semantics (the rounding of every step is part of the
 * result).  One thread; meant for data-independent clocks that are computed once and kept. */
int32_t dgc_clock_accum(dgc_ctx *ctx, float incr, float min, float max, float state0, int32_t T, float *out_dev);
/* The control playhead of the batched harmonic synth (Examples/HarmonicE2E/Synth.swift:57-70):
 * clip(accum((F-1)/(T-1), 0, F-1), 0, F-1-1e-4).  Cached per (F, T) inside the context. */
int32_t dgc_playhead(dgc_ctx *ctx, int32_t F, int32_t T, const float **out_dev);

/* ---- oscillator bank ----------------------------------------------------------------------------
 * How the phase of a stateful phasor is carried across the time axis. */
enum {
  /* frac((f/sr) * n): deterministicPhasor (Sources/DGen/Emit+State.swift:370-387); constant f only */
  DGC_PHASE_DETERMINISTIC = 0,
  /* the reference's recurrence, one single-precision add + wrap per sample, carried serially by
   * one thread per (voice, partial): bit-identical phases (Emit+State.swift:322-369) */
  DGC_PHASE_SEQUENTIAL = 1,
  /* frame-parallel: increments are summed exactly (64-bit fixed point) by a prefix scan across
   * chunks of 64 frames; inside a chunk the single-precision recurrence is followed.  Differs from
   * SEQUENTIAL only by the rounding drift the serial recurrence accumulates across chunks. */
  DGC_PHASE_SCAN = 2,
  /* frame-parallel, one scan per VOICE instead of one per partial: the harmonic bank's partials are multiples
   * k * f0 of one fundamental, so the running sum A[n] = sum_{m<n} f0[m]/sr is kept once per voice in 64-bit
   * fixed point and partial k reads its phase as k * A[n] (mod 1), an exact integer product.  Against SCAN
   * this also drops the rounding of every partial's own increment fl(fl(k*f0)/sr); measured against the
   * step-by-step recurrence both stay inside the 1e-4 sample tolerance (harmonic bank only). */
  DGC_PHASE_FUNDAMENTAL = 3
};

/* Constant-frequency bank summed to mono: audio[n] = sum_k sin(phase_k[n]*2pi) * amp[k].
 * replaces: phasor/deterministicPhasor + sin + mul + sum (Emit+State.swift:322-387,
 * Sources/DGen/Renderer/CRenderer.swift:825-827). */
int32_t dgc_osc_bank_const(dgc_ctx *ctx, const float *freq_dev, const float *amp_dev, int32_t K, int32_t T,
                           float sample_rate, int32_t phase_mode, float *audio_dev);

typedef struct dgc_harmonic_params {
  int32_t B;            /* voices */
  int32_t T;            /* frames */
  int32_t K;            /* partials per voice (1..512) */
  int32_t F;            /* control frames */
  float sample_rate;
  float harmonic_scale; /* harmonicPathScale */
  int32_t phase_mode;   /* DGC_PHASE_SEQUENTIAL, DGC_PHASE_SCAN or DGC_PHASE_FUNDAMENTAL */
  int32_t accumulate;   /* 0: audio = harmonics ; 1: audio += harmonics */
} dgc_harmonic_params;

/* Harmonic branch of HarmonicSynth.renderBatchedSignal (Examples/HarmonicE2E/Synth.swift:47-95):
 * sampleRow of f0/uv/gain [F][B] and amps [F][B][K] at the playhead (Emit+RowSelection.swift:145-213),
 * Nyquist mask + renormalise (Synth.swift:161-170), stateful phasor of k*f0, sin, weighted sum over
 * partials, times gain*uv*scale.  audio is [B][T].
 * scratch: needs dgc_harmonic_scratch_floats(p) floats of device memory (phase anchors and the
 * per-sample fundamental); pass NULL to let the context keep a buffer of its own. */
uint64_t dgc_harmonic_scratch_floats(const dgc_harmonic_params *p);
int32_t dgc_harmonic_render(dgc_ctx *ctx, const dgc_harmonic_params *p, const float *f0_dev, const float *uv_dev,
                            const float *amps_dev, const float *gain_dev, float *scratch_dev, float *audio_dev);

typedef struct dgc_fir_params {
  int32_t B, T, F;
  int32_t taps;        /* FIR length (1..1024); tap taps-1 multiplies the current sample */
  float scale;         /* 0.12 * noisePathScale in the reference */
  int32_t accumulate;  /* 0: audio = branch ; 1: audio += branch */
} dgc_fir_params;

/* Noise branch (Synth.swift:97-101): per-sample interpolated FIR over buffer(size: taps) of the
 * noise input: y[n] = (sum_i x[n-taps+1+i] * lerp(taps_tab)[i]) * lerp(noise_gain) * scale.
 * noise [B][T], taps_tab [F][B][taps], noise_gain [F][B]. */
int32_t dgc_fir_noise(dgc_ctx *ctx, const dgc_fir_params *p, const float *noise_dev, const float *taps_dev,
                      const float *noise_gain_dev, float *audio_dev);

/* Signal.noise() on the device, frame-parallel (jump-ahead of the generator's linear map, then stepping).
 * replaces: the `noise` op -- xorshift32 (13, 17, 5), state bit-stored in a cell, a zero state reseeded to 1,
 * value = state / 2^32 in (0, 1) (Sources/DGen/Renderer/CRenderer.swift:660-695).
 *   DGC_NOISE_STREAM    out[b][n] = value n of the ONE reference stream started from `seed`, bit for bit, the same for
 *                       every voice (Signal.noise().buffer(size:).expand([B, size]), Examples/HarmonicE2E/Synth.swift:97-98);
 *                       sigma is ignored;
 *   DGC_NOISE_GAUSSIAN  white N(0, sigma) per voice, for the synthetic harmonic+noise workload (no reference
 *                       counterpart): voice b runs its own xorshift32 stream from a state hashed from (seed, b);
 *                       frame n maps values 2n and 2n+1 of it through Box-Muller, sigma sqrt(-2 ln u1) cos(2 pi u2). */
enum { DGC_NOISE_STREAM = 0, DGC_NOISE_GAUSSIAN = 1 };
int32_t dgc_noise_fill(dgc_ctx *ctx, uint32_t seed, int32_t mode, int32_t B, int32_t T, float sigma, float *out_dev);

/* taps[r][i] = sum_j W[i][j] * bands[r][j]  (rows r = F*B, W is [taps][nbands]): the linear map
 * from band magnitudes to zero-phase FIR taps used by the synthetic harmonic+noise workload. */
int32_t dgc_bands_to_taps(dgc_ctx *ctx, const float *bands_dev, const float *w_dev, int32_t rows, int32_t nbands,
                          int32_t taps, float *taps_dev);

/* ---- backward of the synthesis w.r.t. the controller outputs -------------------------------------
 * Gradient of the harmonic branch w.r.t. the amplitude table: g_amps [F][B][K] from g_audio [B][T].
 * replaces: the backward of sampleRow + mul + sumAxis + tensorAccumulate
 * (Sources/DGen/Emit+RowSelection.swift:215-330, Sources/DGen/Emit+State.swift:50-115); the phasor
 * input is data (no gradient), as in the HarmonicE2E trainer.  Fixed summation order, no atomics. */
uint64_t dgc_harmonic_bwd_scratch_floats(const dgc_harmonic_params *p);
int32_t dgc_harmonic_render_bwd(dgc_ctx *ctx, const dgc_harmonic_params *p, const float *f0_dev, const float *uv_dev,
                                const float *amps_dev, const float *gain_dev, const float *g_audio_dev,
                                float *scratch_dev, float *g_amps_dev);
/* The same, for a caller that has just rendered the forward with dgc_harmonic_render on the same p, f0, uv and
 * gain and passed it scratch_dev (sized with dgc_harmonic_bwd_scratch_floats): the per-sample tracks and
 * phase anchors the forward left in that scratch are used as they are instead of being computed again; in
 * DGC_PHASE_FUNDAMENTAL mode so are the two per-frame sums the forward divided by (a forward call that is given a
 * scratch leaves them there), and amps_dev is then not read.  The amplitudes must be the forward's.
 * The caller guarantees that the scratch was not written in between.  No reference counterpart (the
 * reference recomputes the forward inside its backward kernels). */
int32_t dgc_harmonic_render_bwd_prepared(dgc_ctx *ctx, const dgc_harmonic_params *p, const float *f0_dev,
                                         const float *uv_dev, const float *amps_dev, const float *gain_dev,
                                         const float *g_audio_dev, float *scratch_dev, float *g_amps_dev);
/* Gradient of the harmonic branch w.r.t. the fundamental table: g_f0 [F][B] from g_audio [B][T], through the
 * phases: dL/dfreq_k[n] = (1/sr) * sum_{m>n} dL/dphi_k[m] (exclusive reverse scan; the wrap is the identity,
 * the Nyquist comparison has no gradient), freq_k = k * sampleRow(f0).
 * replaces: temporalGradStore / temporalGradScan / temporalGradRead of the phasor
 * (Sources/DGen/Gradients.swift:216-261, Sources/DGen/Emit+TemporalGradient.swift:15-110) chained with the
 * backward of sin, mul, sum and sampleRow. */
uint64_t dgc_harmonic_f0_bwd_scratch_floats(const dgc_harmonic_params *p);
int32_t dgc_harmonic_f0_bwd(dgc_ctx *ctx, const dgc_harmonic_params *p, const float *f0_dev, const float *uv_dev,
                            const float *amps_dev, const float *gain_dev, const float *g_audio_dev,
                            float *scratch_dev, float *g_f0_dev);
/* The scan alone, for E rows of T frames (not in place), walking n = T-1 .. 0 from carry = 0:
 *     active = reset[n] > 0 ? 0 : carry ;  out[e][n] = scale * active ;  carry = g[e][n] + active
 * Without resets that is out[e][n] = scale * sum_{m>n} g[e][m]; a reset at frame r cuts the sum for the frames
 * before r AFTER g[r] (the gradient of the pre-update output still enters frame r) and makes out[r] = 0.
 * reset_dev [T] is one signal shared by all rows (> 0 = reset), or NULL for none.
 * replaces: temporalGradScan + temporalGradRead (Emit+TemporalGradient.swift:54-110);
 * scale = 1/sampleRate for a phasor, 1 for an accum. */
int32_t dgc_temporal_grad_scan(dgc_ctx *ctx, const float *g_dev, const float *reset_dev, int32_t E, int32_t T,
                               float scale, float *out_dev);
/* Gradient of the noise branch w.r.t. the tap table: g_taps [F][B][taps] from g_audio [B][T]. */
int32_t dgc_fir_noise_bwd(dgc_ctx *ctx, const dgc_fir_params *p, const float *noise_dev, const float *noise_gain_dev,
                          const float *g_audio_dev, float *g_taps_dev);
/* Controller output heads: z [M][K+NB] -> amps [M][K] = softplus(z[:, :K]) / (row sum + 1e-6), the reference
 * decoder's harmonic head (Examples/HarmonicE2E/Model.swift:102-106), and bands [M][NB] = sigmoid(z[:, K:]), the
 * band-magnitude head of the synthetic harmonic+noise configuration (the reference decoder emits FIR taps and two
 * gains instead, Model.swift:107-113); and backward. */
int32_t dgc_hn_heads_fwd(dgc_ctx *ctx, const float *z_dev, int32_t M, int32_t K, int32_t NB, float *amps_dev,
                         float *bands_dev);
int32_t dgc_hn_heads_bwd(dgc_ctx *ctx, const float *z_dev, const float *g_amps_dev, const float *g_bands_dev,
                         int32_t M, int32_t K, int32_t NB, float *gz_dev);

/* ---- linear recurrences -------------------------------------------------------------------------
 * y[n] = x[n] + a*y[n-1] per voice, chunked parallel scan over time.
 * replaces: historyRead/historyWrite feedback (Sources/DGen/Emit+State.swift:150-224). x,y [B][T]. */
int32_t dgc_onepole_fwd(dgc_ctx *ctx, const float *x_dev, int32_t B, int32_t T, float a, float *y_dev);

/* The same filter continuing from, and leaving behind, the history cell: state_dev [B] holds y[-1] of every voice on
 * entry and y[T-1] on return, so consecutive calls over consecutive blocks of a stream give the output of one call
 * over the whole stream (the reference keeps its cells between realize() calls, preserveState,
 * Sources/DGenLazy/Realize.swift:551-553).  state_dev NULL = start from rest and keep nothing (dgc_onepole_fwd). */
int32_t dgc_onepole_fwd_state(dgc_ctx *ctx, const float *x_dev, int32_t B, int32_t T, float a, float *state_dev,
                              float *y_dev);

/* The same filter for callers that must not allocate.  No counterpart in the reference: it exists
 * because a real-time audio thread (a plug-in render callback, a driver I/O thread) cannot call
 * cudaMalloc -- it may block without bound -- and creating or growing a dgc_ctx does.  This call takes
 * no context and allocates nothing, on the host or on the device: its chunk-carry scratch is a fixed
 * 256 KiB array inside the library's device image, present on every GPU that loads the library until
 * the process exits.
 *   limit     B * ceil(T / 2048) <= DGC_ONEPOLE_STATIC_MAX_CHUNKS (and B <= 65535); larger requests
 *             return DGC_ERR_INVALID with the reason in err_buf (err_buf may be NULL).
 *   set-up    the first call on each device looks up the array's device address
 *             (cudaGetSymbolAddress) with that device current; make that first call before any
 *             stream capture begins.  Later calls only launch kernels on `cuda_stream`
 *             (a cudaStream_t; NULL = default stream) of the CURRENT device and take no lock (the
 *             resolved address is read with one atomic load).
 *   in place  x_dev == y_dev is allowed: every thread reads its run of samples before it writes it.
 *   sharing   all calls on a device use the same array, which keeps the last call's contents; the
 *             filter overwrites every slot before reading it, so nothing needs clearing, but two
 *             calls that overlap on the GPU (different streams, no ordering) race: serialise them. */
#define DGC_ONEPOLE_STATIC_MAX_CHUNKS 32768
int32_t dgc_onepole_fwd_static(void *cuda_stream, const float *x_dev, int32_t B, int32_t T, float a, float *y_dev,
                               char *err_buf, uint32_t err_len);

/* Backward of the one-pole filter (the adjoint of historyRead / historyWrite feedback, Sources/DGen/Gradients.swift:765-778):
 * lam[n] = gy[n] + a lam[n+1], the same scan reversed in time; grad_x = lam [B][T]; grad_a_dev [B] (optional, needs
 * the forward output y_dev) = sum_n lam[n] y[n-1], the derivative with respect to the feedback coefficient. */
int32_t dgc_onepole_bwd(dgc_ctx *ctx, const float *y_dev, const float *gy_dev, int32_t B, int32_t T, float a,
                        float *grad_x_dev, float *grad_a_dev);

typedef struct dgc_biquad_params {
  int32_t B, T, L;   /* voices, frames, lanes */
  float gain;
  float mode;        /* Graph.biquad's selector: 0 low-pass, 1 high-pass, 2 / 3 band-pass (constant skirt / peak
                        gain), 4 all-pass, 5 notch, 6 high shelf, 7 low shelf (the shelves take their amount from
                        `gain`: A = sqrt(|gain|)) */
} dgc_biquad_params;

/* Device scratch (floats) the biquad entry points need: backward 0 = dgc_biquad_fwd, 1 = dgc_biquad_mse_bwd and
 * dgc_biquad_bwd without the input gradient, 2 = dgc_biquad_bwd with it. */
uint64_t dgc_biquad_scratch_floats(const dgc_biquad_params *p, int32_t backward);
/* Tensor biquad bank (Sources/DGen/HigherOps.swift:401-570): x [B][T] shared by L lanes with
 * per-lane cutoff/q; y [B][T][L].  scratch_dev NULL = context-owned buffer. */
int32_t dgc_biquad_fwd(dgc_ctx *ctx, const dgc_biquad_params *p, const float *x_dev, const float *cutoff_dev,
                       const float *q_dev, float *scratch_dev, float *y_dev);
/* The bank continuing from, and leaving behind, Graph.biquad's four history cells (HigherOps.swift:408-437):
 * state_dev [B][4][L] = y[n-1], y[n-2], x[n-1], x[n-2] per voice and lane (the x rows hold the shared input's
 * history: equal across lanes, the kernels read the first lane of a group).  Consecutive calls over consecutive
 * blocks continue the recurrence exactly (preserveState, Sources/DGenLazy/Realize.swift:551-553); calling it block
 * by block with NEW cutoff / q per block is the control-rate form of the reference's per-frame coefficient
 * evaluation (coefficients constant inside a block, state carried across).  state_dev NULL = dgc_biquad_fwd. */
int32_t dgc_biquad_fwd_state(dgc_ctx *ctx, const dgc_biquad_params *p, const float *x_dev, const float *cutoff_dev,
                             const float *q_dev, float *scratch_dev, float *state_dev, float *y_dev);
/* Reverse-time pass (BPTT, Sources/DGen/Gradients.swift:765-778,
 * Sources/DGen/Blocks/Emission/BPTTEmission.swift:471-518) for loss = loss_scale * sum (y - target)^2:
 * gradients w.r.t. the per-lane cutoff and q, summed over voices and frames; loss_dev gets the loss.
 * y, target [B][T][L]. */
int32_t dgc_biquad_mse_bwd(dgc_ctx *ctx, const dgc_biquad_params *p, const float *x_dev, const float *cutoff_dev,
                           const float *q_dev, const float *y_dev, const float *target_dev, float loss_scale,
                           float *scratch_dev, float *grad_cutoff_dev, float *grad_q_dev, double *loss_dev);
/* The same reverse-time pass for an ARBITRARY loss: gy_dev [B][T][L] is dL/dy.  Gradients w.r.t. cutoff and q as
 * above; grad_x_dev [B][T] (optional) receives dL/dx, the sum over lanes of the transposed filters applied to gy
 * (a second reverse sweep from each chunk's resolved terminal adjoint). */
int32_t dgc_biquad_bwd(dgc_ctx *ctx, const dgc_biquad_params *p, const float *x_dev, const float *cutoff_dev,
                       const float *q_dev, const float *y_dev, const float *gy_dev, float *scratch_dev,
                       float *grad_cutoff_dev, float *grad_q_dev, float *grad_x_dev);


/* ---- hop-gated spectral blocks ------------------------------------------------------------------
 * buffer(size:N, hop:) -> FFT -> magnitude for V signals of T frames: mags [V][H][N/2+1],
 * H = ceil(T/hop), window element i of hop frame f = x[f-N+1+i] * window[i] (window NULL = none).
 * replaces: bufferView + acceleratedFFT/tensorFFT + sqrt(re^2+im^2)
 * (HigherOps.swift:738-792, Emit+AcceleratedFFT.swift:16-112, DGenHostSupport.c:10-30). */
int32_t dgc_stft_mag(dgc_ctx *ctx, const float *x_dev, int32_t V, int32_t T, int32_t N, int32_t hop,
                     const float *window_dev, float *mags_dev);

/* buffer(size:N, hop:) -> FFT with ALL N bins kept, split real / imaginary as the reference's spectrum tensors:
 * re_dev, im_dev [V][H][N], H = ceil(T/hop); window as for dgc_stft_mag.
 * replaces: bufferView + acceleratedFFT / tensorFFT (HigherOps.swift:738-792, Emit+AcceleratedFFT.swift:16-112,
 * HigherOps+FFT.swift:16-123).  scratch_dev: dgc_stft_scratch_floats(.., 0) floats or NULL (context scratch). */
uint64_t dgc_stft_scratch_floats(int32_t V, int32_t T, int32_t N, int32_t hop, int32_t inverse);
int32_t dgc_stft_fwd(dgc_ctx *ctx, const float *x_dev, int32_t V, int32_t T, int32_t N, int32_t hop,
                     const float *window_dev, float *scratch_dev, float *re_dev, float *im_dev);

/* IFFT (scaled by 1/N, real part kept) -> * window * gain -> overlapAdd at `hop` into [V][T]; the spectra need not be
 * Hermitian (a phase vocoder's are not): the real part of the inverse transform is what the reference keeps.
 * replaces: acceleratedIFFT / tensorIFFT + overlapAdd (Emit+AcceleratedFFT.swift:16-112, Emit+FFT.swift:6-62).
 * scratch_dev: dgc_stft_scratch_floats(.., 1) floats or NULL.  accumulate != 0: out += result. */
int32_t dgc_istft_ola(dgc_ctx *ctx, const float *re_dev, const float *im_dev, int32_t V, int32_t T, int32_t N,
                      int32_t hop, const float *window_dev, float gain, float *scratch_dev, int32_t accumulate,
                      float *out_dev);

/* partitionedConvolve (Sources/DGenLazy/SpectralTensorOps.swift:204-254,
 * Emit+PartitionedConvolution.swift:26-113, Emit+FFT.swift:6-62): V signals [V][T], one IR; periodic
 * Hann analysis and synthesis windows, IFFT scaled by 1/N, overlap-add at `hop`.
 * scratch_dev: dgc_partconv_scratch_floats() floats, or NULL for a context-owned buffer.
 * accumulate != 0: out += result (dry + wet mix into a buffer that already holds the dry signal). */
uint64_t dgc_partconv_scratch_floats(int32_t V, int32_t T, int32_t ir_len, int32_t N, int32_t hop);
int32_t dgc_partconv(dgc_ctx *ctx, const float *x_dev, int32_t V, int32_t T, const float *ir_dev, int32_t ir_len,
                     int32_t N, int32_t hop, float gain, float *scratch_dev, int32_t accumulate, float *out_dev);

/* Backward of dgc_partconv (linear in x and in ir): g_x [V][T] (overwritten, or += when accumulate_gx)
 * and/or g_ir [ir_len]; pass NULL for the one that is not needed.  The reference defines no backward
 * for this op (Sources/DGen/Gradients.swift:1156-1164): this is the exact adjoint of the forward. */
uint64_t dgc_partconv_bwd_scratch_floats(int32_t V, int32_t T, int32_t ir_len, int32_t N, int32_t hop);
int32_t dgc_partconv_bwd(dgc_ctx *ctx, const float *x_dev, int32_t V, int32_t T, const float *ir_dev, int32_t ir_len,
                         int32_t N, int32_t hop, float gain, const float *g_out_dev, float *scratch_dev,
                         int32_t accumulate_gx, float *g_x_dev, float *g_ir_dev);

/* ---- multi-scale spectral loss ------------------------------------------------------------------ */
#define DGC_MSS_MAX_SCALES 8
typedef struct dgc_mss_params {
  int32_t B, T;
  int32_t nscales;
  int32_t sizes[DGC_MSS_MAX_SCALES]; /* powers of two, 16..4096 */
  int32_t hop_div;                   /* hop = size / hop_div */
  float w_lin, w_log;                /* weights of the L1 linear / L1 log-magnitude terms */
} dgc_mss_params;

/* spectralLossFFTBatched forward for every scale, linear and log-magnitude terms from one FFT
 * (HigherOps.swift:165-263, Emit+SpectralLoss.swift:719-938, Examples/HarmonicE2E/Trainer.swift:538-588):
 * loss = sum_scales (w_lin*lin_s + w_log*log_s) / nscales / T, each term the sum over hop frames of
 * the batch mean.  pred/target [B][T].  loss_dev receives one double.
 * partial_dev (optional) receives per (scale, hop frame, voice) sums: lin then log, see
 * dgc_mss_partial_floats(). */
uint64_t dgc_mss_partial_floats(const dgc_mss_params *p);
int32_t dgc_mss_loss_fwd(dgc_ctx *ctx, const dgc_mss_params *p, const float *pred_dev, const float *target_dev,
                         float *partial_dev, double *loss_dev);
/* Backward: d loss / d pred, [B][T] (Sources/DGen/Gradients.swift:1038-1142,
 * Emit+SpectralLoss.swift:940-1325), recomputing the spectra instead of storing them; `upstream` is
 * d objective / d loss.  grad is overwritten.  Bit-reproducible (no atomics). */
int32_t dgc_mss_loss_bwd(dgc_ctx *ctx, const dgc_mss_params *p, const float *pred_dev, const float *target_dev,
                         float upstream, float *grad_pred_dev);

/* ---- controller -------------------------------------------------------------------------------
 * C[M][N] = act(A[M][K] * W[K][N] + bias[N]); act: 0 none, 1 tanh; bias may be NULL when act == 0.
 * Row-major, full fp32.  ct_dev (optional, may be NULL) receives a second, transposed copy C^T [N][M] of the
 * output: handing it to dgc_linear_bwd of the NEXT layer as at_dev lets that layer's weight gradient run on
 * the faster both-operands-contiguous matmul path.  replaces: matmul -> mul + sumAxis / gemm
 * (Sources/DGen/Tensor.swift:1195-1230, Sources/DGen/Emit+GEMM.swift). */
int32_t dgc_linear_fwd(dgc_ctx *ctx, const float *a_dev, const float *w_dev, const float *bias_dev, int32_t M,
                       int32_t K, int32_t N, int32_t act, float *c_dev, float *ct_dev);
/* Backward of the layer above: dZ = dC * act'(C) (written to dz_dev [M][N]), dW[K][N] = A^T dZ,
 * dbias[N] = column sums of dZ (optional), dA[M][K] = dZ W^T (optional).  at_dev (optional, may be NULL) is
 * A^T [K][M], see dgc_linear_fwd; the result does not depend on whether it is given beyond the rounding of a
 * different summation order.  Sums run in a fixed order
 * (replaces tensorAccumulate, Sources/DGen/Emit+State.swift:50-115). */
int32_t dgc_linear_bwd(dgc_ctx *ctx, const float *a_dev, const float *w_dev, const float *c_dev, const float *dc_dev,
                       int32_t M, int32_t K, int32_t N, int32_t act, float *dz_dev, float *da_dev, float *dw_dev,
                       float *dbias_dev, const float *at_dev);

/* How many matrix products this context has sent to each kernel family since it was created: out4[0] SIMT register
 * tiles (small products), [1] tcgen05 kernel for any operand orientation, [2] tcgen05 asynchronous pipeline (both
 * operands contiguous along the reduction), [3] the same with 128 x 256 output tiles.  For tests and profiling: a shape
 * that silently left the tensor cores shows here.  No reference counterpart. */
int32_t dgc_gemm_path_counts(dgc_ctx *ctx, int64_t *out4);

/* Adam step on device (Sources/DGenLazy/Optimizers.swift:164-243: bias-corrected, eps outside the
 * square root, the reference's operation order); t is the 1-based step index. */
int32_t dgc_adam_step(dgc_ctx *ctx, float *theta_dev, const float *grad_dev, float *m_dev, float *v_dev, uint64_t n,
                      int32_t t, float lr, float beta1, float beta2, float eps);

/* The same step with the step index kept on the device: *t_dev (int32, 0 before the first step) is incremented by
 * the call and the bias corrections are evaluated on the device into corr_dev[2], so a recorded step (dgc_graph_*)
 * advances the index on every replay. */
int32_t dgc_adam_step_counted(dgc_ctx *ctx, float *theta_dev, const float *grad_dev, float *m_dev, float *v_dev,
                              uint64_t n, int32_t *t_dev, float *corr_dev, float lr, float beta1, float beta2,
                              float eps);

/* Sum over frames of a per-frame tensor: out[e] (+)= scale * sum_n x[n][e], x_dev [T][E].  The accumulation of
 * per-frame parameter gradients into the parameter's gradient cell (tensorAccumulate / memoryAccumulate,
 * Sources/DGen/Emit+State.swift:50-115; read back by Sources/DGenLazy/Backward.swift:132-165), in a fixed order
 * (double-precision segment sums): the result does not depend on scheduling.  accumulate != 0 adds to out. */
int32_t dgc_reduce_frames(dgc_ctx *ctx, const float *x_dev, int64_t T, int64_t E, float scale, int32_t accumulate,
                          float *out_dev);

/* Output sanitiser: out[i] = in[i] when its IEEE-754 exponent field is not all ones, else +0.0f (NaN and
 * +-Inf become 0; denormals, -0.0 and every finite value pass through bit for bit).  in_dev == out_dev is
 * allowed.  Replaces dgen_sanitize_f32 / dgen_sanitize_f32x4 applied at every `output` store
 * (toolchain/include/dgen_runtime.h:59-84, Sources/DGen/Renderer/CRenderer.swift:1021-1039). */
int32_t dgc_sanitize(dgc_ctx *ctx, const float *in_dev, uint64_t n, float *out_dev);

/* ---- ring and hold ops ------------------------------------------------------------------------------
 * The reference runs these frame by frame in sequential blocks because they read and write a memory cell;
 * here every (frame, lane) element is computed independently from the input and from the cell contents at
 * the start of the call, and the cells are rewritten at the end so consecutive calls continue seamlessly.
 * State pointers may be NULL: the cells then start at zero and are not kept.  x and y must not alias. */

/* Per-lane interpolated delay lines with one shared write head: tensorDelay
 * (Sources/DGen/HigherOps+DelayLine.swift:33-65; emission Sources/DGen/Emit.swift:331-403).
 * x_dev, y_dev [T][lanes]; delay in samples, clamped to [0, max_delay - 1], linear interpolation between the
 * two bracketing past samples (a delay of 0 returns the current sample).
 * delay_mode: 0 = delay_dev[0] for the whole call, 1 = [T], 2 = [T][lanes], 3 = [lanes].
 * ring_dev [lanes][max_delay] (lane-major, as the reference's buffer cell), head_dev 1 float (write position). */
int32_t dgc_delay_line(dgc_ctx *ctx, const float *x_dev, const float *delay_dev, int32_t delay_mode, int64_t T,
                       int32_t lanes, int32_t max_delay, float *ring_dev, float *head_dev, float *y_dev);

/* Delay of an [N] spectrum by whole or fractional hop boundaries: spectrumDelay / spectrumDelayMod
 * (Sources/DGen/HigherOps+SpectrumDelay.swift:20-135; emission Sources/DGen/Emit.swift:405-512).
 * spec_dev, out_dev [H][N]: one row per hop boundary.  delay_dev NULL: the row of exactly `hops` boundaries ago.
 * delay_dev [H]: delay in hops, clamped to [0, hops], linear interpolation between floor and floor + 1 ago.
 * ring_dev [hops + 1][N], row_dev 1 float (next write row). */
int32_t dgc_spectrum_delay(dgc_ctx *ctx, const float *spec_dev, const float *delay_dev, int64_t H, int32_t N,
                           int32_t hops, float *ring_dev, float *row_dev, float *out_dev);

/* Sample and hold: y[n][e] = value[n][e] where cond > 0, else the value held from the most recent such frame
 * (state_dev [lanes] before the first; updated to the last output).  latch
 * (Sources/DGen/Definitions.swift:104-113 scalar, Sources/DGen/Emit+State.swift:225-262 tensor,
 * Sources/DGen/HigherOps+Latch.swift:31-57).  cond_mode: 1 = cond_dev [T] shared by the lanes, 2 = [T][lanes].
 * scratch_dev: dgc_latch_scratch_floats floats, or NULL to use context scratch. */
uint64_t dgc_latch_scratch_floats(int64_t T, int32_t lanes);
int32_t dgc_latch(dgc_ctx *ctx, const float *value_dev, const float *cond_dev, int32_t cond_mode, int64_t T,
                  int32_t lanes, float *state_dev, float *scratch_dev, float *y_dev);

/* Feed-forward compressor with soft knee and attack / release smoothing of the gain reduction in dB:
 * Graph.compressor (Sources/DGen/HigherOps.swift:566-651).  x_dev, y_dev [B][T]; sidechain_dev [B][T] or NULL
 * (detector = the input); state_dev [B] = previous smoothed gain reduction (the history cell), or NULL. */
typedef struct dgc_compressor_params {
  int32_t B;
  int64_t T;
  float ratio, threshold, knee; /* threshold and knee in dB */
  float attack, release;        /* seconds */
  float sample_rate;
} dgc_compressor_params;
int32_t dgc_compressor(dgc_ctx *ctx, const dgc_compressor_params *p, const float *x_dev, const float *sidechain_dev,
                       float *state_dev, float *y_dev);

/* Phase-vocoder pitch shift of a stream of N-bin spectra: phaseVocoder
 * (Sources/DGen/HigherOps+PhaseVocoder.swift:15-88; emission Sources/DGen/Emit+PhaseVocoder.swift:6-118).
 * re_dev, im_dev, out_re_dev, out_im_dev [V][H][N] (one row per hop boundary, all N bins).
 * ratio_mode: 0 = ratio_dev[0], 1 = ratio_dev [H] shared by the voices, 2 = [V][H]; ratios below 1e-4 are raised to it.
 * state_dev [V][2N+1] = previous analysis phase [N], synthesis phase [N], started flag; NULL = a fresh stream.
 * scratch_dev: dgc_phase_vocoder_scratch_floats floats or NULL. */
uint64_t dgc_phase_vocoder_scratch_floats(int32_t V, int64_t H, int32_t N);
int32_t dgc_phase_vocoder(dgc_ctx *ctx, const float *re_dev, const float *im_dev, const float *ratio_dev,
                          int32_t ratio_mode, int32_t V, int64_t H, int32_t N, int32_t hop, float *state_dev,
                          float *scratch_dev, float *out_re_dev, float *out_im_dev);

/* ---- step replay ---------------------------------------------------------------------------------------
 * Record everything enqueued through this context between dgc_graph_begin and dgc_graph_end (work the host puts on
 * other streams that fork from and join back into the context's stream is recorded with it), then replay it with
 * one dgc_graph_launch per step.
 * replaces: the per-step graph rebuild, recompilation and tensor re-upload of the reference's training loop
 * (Sources/DGenLazy/Backward.swift:225, Sources/DGenLazy/Realize.swift:285-290, Sources/DGenLazy/LazyGraph.swift:171-234).
 * The context must be bound to a non-default stream; run the step once before recording it, so that nothing inside
 * the recording allocates; values passed by value are frozen into the recording -- refill input buffers in place and
 * use dgc_adam_step_counted.  dgc_graph_end reports an invalidated recording as DGC_ERR_CUDA with the reason.
 * A recording holds the addresses of the context's own buffers (scratch, staging, transposed operands).  If a
 * call made AFTER the recording needs a larger one, the context reallocates it; dgc_graph_launch notices and
 * returns DGC_ERR_INVALID without launching anything: record the step again.
 * dgc_allreduce_sum on a context with a communicator is refused (DGC_ERR_INVALID) between dgc_graph_begin and
 * dgc_graph_end: record forward + backward, exchange call by call, record the update as a second step. */
typedef struct dgc_graph dgc_graph;
int32_t dgc_graph_begin(dgc_ctx *ctx);
int32_t dgc_graph_end(dgc_ctx *ctx, dgc_graph **out);
uint64_t dgc_graph_nodes(const dgc_graph *g);
int32_t dgc_graph_launch(dgc_ctx *ctx, dgc_graph *g);
int32_t dgc_graph_destroy(dgc_graph *g);

/* ---- generated blocks -------------------------------------------------------------------------------
 * Device code the host's renderer emits for elementwise blocks that no primitive above covers.
 * replaces: compiling the C renderer's source and loading it (Sources/DGen/Runtime.swift:291-311) and
 * the call of the generated `process` symbol (toolchain/include/dgen_runtime.h:282-290).
 * dgc_module_load takes a cubin for sm_100a or NUL-terminated PTX; dgc_module_compile takes CUDA C and
 * compiles it in process with NVRTC (found at run time; DGC_NVRTC_PATH overrides the search).  Kernels are
 * extern "C" __global__ functions, launched on the context stream with the argument-pointer array of
 * cudaLaunchKernel. */
typedef struct dgc_module dgc_module;
int32_t dgc_module_load(dgc_ctx *ctx, const void *image, uint64_t size, dgc_module **out);
int32_t dgc_module_compile(dgc_ctx *ctx, const char *cuda_source, const char *name, dgc_module **out);
int32_t dgc_module_unload(dgc_module *m);
int32_t dgc_launch(dgc_module *m, const char *kernel_name, const uint32_t grid[3], const uint32_t block[3],
                   uint32_t smem_bytes, void **args);

/* Blocks as op lists: the elementwise subset of the reference's UOps in SSA form (the value of op k is t_k;
 * operands a, b, c are ids of earlier ops, or an arena cell offset for the memory ops), one thread per
 * (frame, element) index i < count.  dgc_block_emit writes the CUDA C of `extern "C" __global__ void
 * name(float *memory, int count)` using the scalar expressions of the reference's C renderer for every op
 * (Sources/DGen/Renderer/CRenderer.swift:484-1040): division / modulo / power by a constant are specialised
 * the same way, comparisons and logic yield 1.0f / 0.0f, gswitch tests `> 0`, OUTPUT sanitises.
 * `needed` receives the size of the source including the terminator; call with out == NULL to size it.
 * dgc_block_compile = emit + dgc_module_compile. */
enum {
  DGC_OP_CONST = 0,      /* imm */
  DGC_OP_LOAD = 1,       /* memory[a + i] */
  DGC_OP_LOAD_SCALAR = 2,/* memory[a] */
  DGC_OP_FRAME_INDEX = 3,/* (float)i */
  DGC_OP_ADD = 10, DGC_OP_SUB, DGC_OP_MUL, DGC_OP_DIV, DGC_OP_MOD, DGC_OP_POW, DGC_OP_MIN, DGC_OP_MAX, DGC_OP_ATAN2,
  DGC_OP_AND, DGC_OP_OR, DGC_OP_XOR, DGC_OP_GT, DGC_OP_GTE, DGC_OP_LTE, DGC_OP_LT, DGC_OP_EQ,
  DGC_OP_ABS = 40, DGC_OP_SIGN, DGC_OP_FLOOR, DGC_OP_CEIL, DGC_OP_ROUND, DGC_OP_SIN, DGC_OP_COS, DGC_OP_TAN,
  DGC_OP_ATAN, DGC_OP_TANH, DGC_OP_EXP, DGC_OP_LOG, DGC_OP_LOG10, DGC_OP_SQRT,
  DGC_OP_GSWITCH = 60,   /* t_a > 0 ? t_b : t_c */
  DGC_OP_STORE = 70,     /* memory[a + i] = t_b */
  DGC_OP_OUTPUT = 71,    /* memory[a + i] = sanitize(t_b) */
  /* sequential form only (one thread per lane e, frames i in order; a = arena cell offset) */
  DGC_OP_LOAD_LANE = 80,        /* memory[a + e]: per-lane, frame-invariant */
  DGC_OP_LOAD_FRAME_LANE = 81,  /* memory[a + i * lanes + e]: frame-aware tensor */
  DGC_OP_STORE_FRAME_LANE = 82, /* memory[a + i * lanes + e] = t_b */
  DGC_OP_HISTORY_READ = 83,     /* content of state cell a (per lane: memory[a + e]) */
  DGC_OP_HISTORY_WRITE = 84,    /* state cell a = t_b (pass-through) */
  DGC_OP_PHASOR = 85,           /* state cell a; frequency t_b, reset t_c, imm = sample rate; value = phase before the update */
  DGC_OP_LATCH = 86,            /* state cell a = t_b where t_c > 0; value = the cell */
  DGC_OP_ACCUM = 87,            /* state cell a; increment t_b, reset t_c, wraps in [0, imm); value = state before the update */
  DGC_OP_NOISE = 88             /* state cell a = xorshift32 state (raw bits); value = new state / 2^32 */
};
typedef struct dgc_uop {
  int32_t op;
  int32_t a, b, c;
  float imm;
} dgc_uop;
int32_t dgc_block_emit(const dgc_uop *ops, int32_t n_ops, const char *kernel_name, char *out, uint64_t out_cap,
                       uint64_t *needed);
int32_t dgc_block_compile(dgc_ctx *ctx, const dgc_uop *ops, int32_t n_ops, const char *kernel_name, dgc_module **out);

/* Blocks with state cells (history feedback, phasor, latch: the reference's sequential blocks,
 * Sources/DGen/Blocks/FeedbackAnalysis.swift:357-365, Sources/DGen/Emit+State.swift:150-369): the same op lists,
 * emitted as `extern "C" __global__ void name(float *memory, int frames, int lanes)` with one thread per tensor
 * lane and the frame loop inside it, in frame order.  In this form i is the FRAME (DGC_OP_LOAD reads a per-frame
 * scalar signal memory[a + i]), the lane-indexed ops above address tensors, and every state cell of a lane lives
 * in a register across the loop (read from memory[a + e] before, written back after), so consecutive calls
 * continue where the last one stopped, as the reference's persistent cells do. */
int32_t dgc_block_emit_sequential(const dgc_uop *ops, int32_t n_ops, const char *kernel_name, char *out,
                                  uint64_t out_cap, uint64_t *needed);
int32_t dgc_block_compile_sequential(dgc_ctx *ctx, const dgc_uop *ops, int32_t n_ops, const char *kernel_name,
                                     dgc_module **out);

/* ---- block plans ---------------------------------------------------------------------------------------
 * What the host's block matcher hands over for one realize() / backward(): the scheduler's blocks in order
 * (Sources/DGen/Blocks/BlockFormation.swift:5-85 partitionIntoBlocks, :1733 determineTensorBlocks), each either a
 * recognised primitive of this library or a generated block (dgc_block_compile), with every buffer given as an
 * OFFSET into one arena, the way the reference's kernels address one flat `memory` through cell offsets
 * (Sources/DGen/Renderer/Renderer.swift:134-143 CompiledKernel, Sources/DGen/Runtime.swift:732-744).
 * dgc_plan_run enqueues the steps on the context stream in order; steps marked stream 1 go to the context's side
 * stream between a DGC_PLAN_FORK (side starts where main stands) and a DGC_PLAN_JOIN (main waits for side), which
 * is how independent blocks -- the harmonic and the noise branch of the synthesiser -- overlap.  A plan can be
 * recorded (dgc_graph_begin / _end around dgc_plan_run) and replayed, except for DGC_PLAN_ALLREDUCE steps.
 *
 * Step arguments: a[] = arena offsets in floats (DGC_PLAN_NONE = absent), i[] = integers, f[] = floats; an
 * offset that receives a double (a loss) must be even and takes two floats.  Per op (names as the entry points):
 *   FORK, JOIN            -
 *   OSC_BANK_CONST        a: freq amp audio                  i: K T phase_mode             f: sample_rate
 *   HARMONIC_RENDER       a: f0 uv amps gain scratch audio   i: B T K F phase_mode accumulate   f: sample_rate scale
 *   BANDS_TO_TAPS         a: bands w taps                    i: rows nbands taps
 *   FIR_NOISE             a: noise taps noise_gain audio     i: B T F taps accumulate      f: scale
 *   ADD                   a: x y out n                       (out = x + y over n floats; out may be x)
 *   COPY                  a: src dst n
 *   ONEPOLE               a: x y state                       i: B T                        f: a
 *   BIQUAD_FWD            a: x cutoff q scratch state y      i: B T L                      f: gain mode
 *   BIQUAD_MSE_BWD        a: x cutoff q y target scratch grad_cutoff grad_q loss   i: B T L   f: gain mode loss_scale
 *   STFT_MAG              a: x window mags                   i: V T N hop
 *   PARTCONV              a: x ir scratch out                i: V T ir_len N hop accumulate    f: gain
 *   PARTCONV_BWD          a: x ir g_out scratch g_x g_ir     i: V T ir_len N hop accumulate_gx f: gain
 *   MSS_LOSS_FWD          a: pred target partial loss        i: B T nscales hop_div size0..    f: w_lin w_log
 *   MSS_LOSS_BWD          a: pred target grad                i: B T nscales hop_div size0..    f: w_lin w_log upstream
 *   LINEAR_FWD            a: A W bias C Ct                   i: M K N act
 *   LINEAR_BWD            a: A W C dC dZ dA dW dbias At      i: M K N act
 *   HEADS_FWD             a: z amps bands                    i: M K NB
 *   HEADS_BWD             a: z g_amps g_bands gz             i: M K NB
 *   HARMONIC_BWD          a: f0 uv amps gain g_audio scratch g_amps   i: B T K F phase_mode prepared   f: sample_rate scale
 *   FIR_BWD               a: noise noise_gain g_audio g_taps i: B T F taps                 f: scale
 *   ALLREDUCE             a: buf n
 *   ADAM                  a: theta grad m v t_cell corr n    f: lr beta1 beta2 eps   (dgc_adam_step_counted: t_cell is one
 *                                                            int32 in the arena, corr two floats)
 *   SANITIZE              a: in out n
 *   BLOCK                 i: kernel_index form count_or_frames lanes   (form 0: name(memory, count), one thread per
 *                                                            index; form 1: name(memory, frames, lanes), one thread per lane)
 */
#define DGC_PLAN_NONE 0xffffffffffffffffull
enum {
  DGC_PLAN_FORK = 0, DGC_PLAN_JOIN, DGC_PLAN_OSC_BANK_CONST, DGC_PLAN_HARMONIC_RENDER, DGC_PLAN_BANDS_TO_TAPS,
  DGC_PLAN_FIR_NOISE, DGC_PLAN_ADD, DGC_PLAN_COPY, DGC_PLAN_ONEPOLE, DGC_PLAN_BIQUAD_FWD, DGC_PLAN_BIQUAD_MSE_BWD,
  DGC_PLAN_STFT_MAG, DGC_PLAN_PARTCONV, DGC_PLAN_PARTCONV_BWD, DGC_PLAN_MSS_LOSS_FWD, DGC_PLAN_MSS_LOSS_BWD,
  DGC_PLAN_LINEAR_FWD, DGC_PLAN_LINEAR_BWD, DGC_PLAN_HEADS_FWD, DGC_PLAN_HEADS_BWD, DGC_PLAN_HARMONIC_BWD,
  DGC_PLAN_FIR_BWD, DGC_PLAN_ALLREDUCE, DGC_PLAN_ADAM, DGC_PLAN_SANITIZE, DGC_PLAN_BLOCK, DGC_PLAN_OP_COUNT
};
typedef struct dgc_plan_step {
  int32_t op;        /* DGC_PLAN_* */
  int32_t stream;    /* 0 = the context stream, 1 = the side stream */
  uint64_t a[10];
  int32_t i[16];
  float f[4];
} dgc_plan_step;
typedef struct dgc_plan {
  const dgc_plan_step *steps;
  int32_t n_steps;
  dgc_module *const *modules;   /* BLOCK steps: i[0] indexes modules and kernels (may be NULL when there are none) */
  const char *const *kernels;
  int32_t n_kernels;
} dgc_plan;
/* Runs steps [first, first + count) of the plan on the arena (count < 0: to the end).  On an error the step index is
 * part of dgc_last_error and nothing after it is enqueued; a side stream that was forked is joined first. */
int32_t dgc_plan_run(dgc_ctx *ctx, dgc_arena *arena, const dgc_plan *plan, int32_t first, int32_t count);

/* The training step of the harmonic+noise model as a plan (Examples/HarmonicE2E/Trainer.swift:247-487: forward ->
 * multi-scale spectral loss -> backward -> optimizer step; Sources/DGenLazy/Backward.swift:174-230,
 * Sources/DGenLazy/Optimizers.swift:164-243), with every tensor at a fixed arena offset:
 *   controller h = tanh(.. tanh(X W0 + b0) ..) (n_trunk layers of `hidden`), z = h Wh + bh, heads (dgc_hn_heads_fwd),
 *   taps = bands Wfs^T, dry = harmonic + FIR noise, out = dry + partitioned_convolve(dry, ir), 6-scale loss,
 *   the backward of all of it into ONE flat gradient vector, all-reduce, Adam.
 * Parameters are one flat vector: W0 [in][hidden], b0, W1, b1, .., Wh [hidden][K + nbands], bh, ir [ir_len].
 * dgc_hn_train_plan fills `layout` (where the host puts inputs and finds outputs) and writes the steps:
 * [0, n_forward_backward) is forward + backward, then one ALLREDUCE step, then one ADAM step.  A host with several
 * ranks records the first range and the ADAM step separately and runs the ALLREDUCE step between the replays. */
typedef struct dgc_hn_train_config {
  int32_t B, T, K, F;        /* local voices, frames, harmonics, control frames */
  float sample_rate;
  int32_t nbands, taps;
  int32_t in_features, hidden, n_trunk;   /* controller: in -> hidden x n_trunk (tanh) -> K + nbands */
  int32_t ir_len, conv_n, conv_hop;       /* learnable impulse response, partition size and hop */
  dgc_mss_params mss;
  int32_t phase_mode;
  int32_t global_voices;     /* voices over all ranks (the loss gradient is scaled by B / global_voices) */
  float lr, beta1, beta2, eps;
} dgc_hn_train_config;
typedef struct dgc_hn_train_layout {
  uint64_t total_floats;     /* arena size */
  uint64_t n_params;
  uint64_t params, grads, adam_m, adam_v, adam_t, adam_corr;
  uint64_t x, f0, uv, gain, noise_gain, noise, w_fs, target;    /* inputs: X [F*B][in], controls [F][B], noise and target [B][T], Wfs [taps][nbands] */
  uint64_t loss;             /* one double (two floats, even offset) */
  uint64_t audio;            /* out [B][T]: dry + reverb */
  int32_t n_steps, n_forward_backward;
} dgc_hn_train_layout;
/* steps may be NULL to size it (layout->n_steps).  Returns DGC_ERR_INVALID when cap is too small. */
int32_t dgc_hn_train_plan(const dgc_hn_train_config *cfg, dgc_hn_train_layout *layout, dgc_plan_step *steps,
                          int32_t cap);

/* ---- gradient exchange between GPUs ------------------------------------------------------------------
 * One process per GPU, one communicator per context (NCCL, found at run time; DGC_NCCL_PATH overrides).
 * Rank 0 creates the id, the host hands its DGC_COMM_ID_BYTES bytes to every rank, every rank calls
 * dgc_comm_init, then dgc_allreduce_sum(buf) leaves the sum over ranks in buf on every rank (in place, on
 * the context stream).  Without a communicator dgc_allreduce_sum is the identity (a world of one).
 * replaces: nothing in the reference (it trains on one device); the buffer is what readGradients collects
 * (Sources/DGenLazy/Backward.swift:132-165). */
#define DGC_COMM_ID_BYTES 128
int32_t dgc_comm_unique_id(uint8_t *id_out);
int32_t dgc_comm_init(dgc_ctx *ctx, int32_t world, int32_t rank, const uint8_t *id);
int32_t dgc_allreduce_sum(dgc_ctx *ctx, float *buf_dev, uint64_t n_floats);
int32_t dgc_comm_destroy(dgc_ctx *ctx);

/* ---- composite steps with host buffers (the call a host makes per batch) ------------------------ */
typedef struct dgc_hn_step {
  dgc_harmonic_params harm;
  dgc_fir_params fir;      /* fir.taps == 0 disables the noise branch */
  dgc_mss_params mss;
  int32_t nbands;          /* > 0: taps are synthesised from bands_host [F][B][nbands] with w_host [taps][nbands] */
  /* Host-buffer entry points only (the device-resident call ignores them):
   * noise_seed != 0 and noise_host == NULL: the noise is generated on the device (dgc_noise_fill with noise_mode and
   * noise_sigma) instead of being uploaded -- the reference generates its noise inside the graph too;
   * target_dev != NULL: the target already lives in device memory ([B][T]) and target_host is not uploaded. */
  uint32_t noise_seed;
  int32_t noise_mode;
  float noise_sigma;
  const float *target_dev;
} dgc_hn_step;

/* Harmonic+noise synthesis forward + multi-scale spectral loss with every buffer in device memory: what a host
 * that keeps its tensors resident calls once per batch.  The harmonic and the noise branch run concurrently on
 * two streams and meet at the loss; the caller's stream (the context stream) is joined before the call returns,
 * so the usual stream order holds for whatever the caller enqueues next.  work_dev: scratch of
 * dgc_hn_forward_loss_work_floats(s) floats, 16-byte aligned.  audio_dev (optional) receives the summed signal.
 * replaces: one realize() of the HarmonicE2E forward graph on resident tensors. */
uint64_t dgc_hn_forward_loss_work_floats(const dgc_hn_step *s);
int32_t dgc_hn_forward_loss(dgc_ctx *ctx, const dgc_hn_step *s, const float *f0_dev, const float *uv_dev,
                            const float *amps_dev, const float *gain_dev, const float *noise_gain_dev,
                            const float *taps_or_bands_dev, const float *w_dev, const float *noise_dev,
                            const float *target_dev, float *work_dev, double *loss_dev, float *audio_dev);

/* Harmonic+noise synthesis forward + multi-scale spectral loss, inputs and result in host memory:
 * uploads the control tables, noise and target, renders, evaluates the loss and returns it.
 * audio_host may be NULL.  replaces: one realize() of the HarmonicE2E forward graph. */
int32_t dgc_hn_forward_loss_host(dgc_ctx *ctx, const dgc_hn_step *s, const float *f0_host, const float *uv_host,
                                 const float *amps_host, const float *gain_host, const float *noise_gain_host,
                                 const float *taps_or_bands_host, const float *w_host, const float *noise_host,
                                 const float *target_host, double *loss_host, float *audio_host);

/* The same step with TWO steps in flight: submit enqueues the uploads (into the slot's own staging area), the step and
 * the read-back of the loss and returns at once; wait blocks until that slot's step has finished and *loss_host (and
 * audio_host) are valid.  While slot 0 computes, the inputs of slot 1 cross PCIe: steady-state throughput is the
 * larger of upload time and compute time instead of their sum.  Host buffers of a slot must stay untouched from
 * submit to wait (pinned memory, or the copies are not asynchronous).  slot is 0 or 1; a slot is reusable after its
 * wait.  Typical loop: submit(i % 2) then wait((i - 1) % 2). */
int32_t dgc_hn_forward_loss_host_submit(dgc_ctx *ctx, const dgc_hn_step *s, const float *f0_host, const float *uv_host,
                                        const float *amps_host, const float *gain_host,
                                        const float *noise_gain_host, const float *taps_or_bands_host,
                                        const float *w_host, const float *noise_host, const float *target_host,
                                        int32_t slot, double *loss_host, float *audio_host);
int32_t dgc_hn_forward_loss_host_wait(dgc_ctx *ctx, int32_t slot);

#ifdef __cplusplus
}
#endif
#endif
