// Composite entry points that take HOST buffers: what a host calls once per batch.  They own a
// device staging area inside the context, enqueue one asynchronous copy per input straight from the
// caller's buffers (full PCIe rate when those are page-locked) on an upload stream, in the order the
// kernels need them, and the kernels on the context stream behind per-group events: the render starts
// as soon as its control tables have landed, while the noise inputs and the target are still in
// flight.  The result returns to host memory.
#include "common.cuh"
#include <cstdlib>
#include <cstring>

namespace {

// device staging area carved into sub-buffers, grown on demand
struct Carver {
  float *base;
  uint64_t used = 0;
  explicit Carver(float *b) : base(b) {}
  float *take(uint64_t n) {
    float *p = base + used;
    used += (n + 63) & ~63ull;  // keep every sub-buffer 256-byte aligned
    return p;
  }
};

int32_t ensure_stage(dgc_ctx *ctx, uint64_t nfloats) {
  if (nfloats <= ctx->stage_floats) return DGC_OK;
  if (ctx->stage_dev) {
    cudaStreamSynchronize(ctx->stream);
    cudaFree(ctx->stage_dev);
    ctx->buffer_generation++;
    ctx->stage_dev = nullptr;
    ctx->stage_floats = 0;
  }
  DGC_CUDA(ctx, cudaMalloc(&ctx->stage_dev, nfloats * sizeof(float)));
  ctx->stage_floats = nfloats;
  return DGC_OK;
}

// out may be the same buffer as a (element i is read before it is written): no restrict on those two
__global__ void add2_kernel(const float *a, const float *__restrict__ b, size_t n, float *out) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __fadd_rn(a[i], b[i]);
}

}  // namespace

DGC_EXPORT uint64_t dgc_hn_forward_loss_work_floats(const dgc_hn_step *s) {
  if (!s || s->harm.B <= 0 || s->harm.T <= 0 || s->harm.F <= 0) return 0;
  const uint64_t nBT = ((uint64_t)s->harm.B * s->harm.T + 63) & ~63ull;
  const uint64_t taps = (s->fir.taps > 0 && s->nbands > 0) ? (((uint64_t)s->harm.F * s->harm.B * s->fir.taps + 63) & ~63ull) : 0;
  return 2 * nBT + taps + 64;
}

// Device-resident forward + loss.  The harmonic branch (track, chunk sums, scan, render) and the noise branch
// (band -> tap map, FIR) share no data until the loss, so they run on two streams: the small or latency-bound
// kernels of one chain (the 64-block phase scan, the band -> tap matmul) and the last waves of the big ones fill
// under the other chain's work.  The loss reads the prediction as the sum of the two branch outputs.
// ev_noise_inputs / ev_target (optional): events after which the noise-branch inputs / the target are in device
// memory (the host-buffer variant uploads them on its own stream while the first kernels already run)
static int32_t hn_forward_loss_impl(dgc_ctx *ctx, const dgc_hn_step *s, const float *f0_dev, const float *uv_dev,
                                    const float *amps_dev, const float *gain_dev, const float *noise_gain_dev,
                                    const float *taps_or_bands_dev, const float *w_dev, const float *noise_dev,
                                    const float *target_dev, float *work_dev, double *loss_dev, float *audio_dev,
                                    cudaEvent_t ev_noise_inputs, cudaEvent_t ev_target) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, s && f0_dev && uv_dev && amps_dev && gain_dev && target_dev && loss_dev && work_dev, "null pointer");
  const int B = s->harm.B, T = s->harm.T, K = s->harm.K, F = s->harm.F;
  DGC_REQUIRE(ctx, B > 0 && T > 0 && K > 0 && F > 0, "size out of range");
  const int NT = s->fir.taps, NB = s->nbands;
  const bool noise = NT > 0;
  if (noise) {
    DGC_REQUIRE(ctx, noise_gain_dev && taps_or_bands_dev && noise_dev, "noise branch needs its inputs");
    DGC_REQUIRE(ctx, s->fir.B == B && s->fir.T == T && s->fir.F == F, "fir shape differs from harmonic shape");
    DGC_REQUIRE(ctx, NB == 0 || w_dev, "band synthesis needs the matrix W");
  }
  DGC_REQUIRE(ctx, s->mss.B == B && s->mss.T == T, "loss shape differs from harmonic shape");
  DGC_REQUIRE(ctx, (((uintptr_t)work_dev) & 15) == 0, "work buffer must be 16-byte aligned");
  const uint64_t nBT = (uint64_t)B * T, nFB = (uint64_t)F * B;
  Carver wc(work_dev);
  float *d_harm = wc.take(nBT), *d_noise = noise ? wc.take(nBT) : nullptr;
  float *d_taps = (noise && NB > 0) ? wc.take(nFB * NT) : const_cast<float *>(taps_or_bands_dev);
  // Size the context scratch for the largest user BEFORE the streams fork: growing it later would free a buffer
  // the other stream may still be reading.
  {
    uint64_t need = dgc_harmonic_scratch_floats(&s->harm), m = dgc_mss_partial_floats(&s->mss) + 4;
    if (m > need) need = m;
    if (!dgc_ctx_scratch(ctx, need)) return DGC_ERR_OOM;
  }
  if (!ctx->aux_stream) {
    DGC_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->aux_stream, cudaStreamNonBlocking));
    DGC_CUDA(ctx, cudaEventCreateWithFlags(&ctx->fork_ev, cudaEventDisableTiming));
    DGC_CUDA(ctx, cudaEventCreateWithFlags(&ctx->join_ev, cudaEventDisableTiming));
  }
  // tables cached per (F, T) are built on first use by a kernel on the current stream: make sure they exist
  // before the streams fork, so that neither branch picks up a table the other one is still writing
  if (!dgc_ctx_row_table(ctx, F, T)) return DGC_ERR_CUDA;
  int32_t rc = DGC_OK;
  cudaStream_t main_stream = ctx->stream;
  bool forked = false;
  // From a few million samples per step on, every big kernel fills the GPU by itself and running the FIR beside the
  // render buys nothing: then only the band -> tap map runs on the side stream, and the FIR follows the render on
  // the caller's stream ADDING into the render's output, which drops the pass that sums the two branches (the sum
  // is the same single-precision add either way: the results are bit-identical).  DGC_HN_FIR=side|serial forces one.
  static const int fir_mode = [] {
    const char *e = getenv("DGC_HN_FIR");
    return !e ? 0 : strcmp(e, "side") == 0 ? 1 : strcmp(e, "serial") == 0 ? 2 : 0;
  }();
  const bool serial_fir = noise && (fir_mode == 2 || (fir_mode == 0 && nBT >= (4ull << 20)));
  if (noise) {
    // fork: the noise branch starts where the caller's stream stands now
    DGC_CUDA(ctx, cudaEventRecord(ctx->fork_ev, main_stream));
    DGC_CUDA(ctx, cudaStreamWaitEvent(ctx->aux_stream, ctx->fork_ev, 0));
    if (ev_noise_inputs) DGC_CUDA(ctx, cudaStreamWaitEvent(ctx->aux_stream, ev_noise_inputs, 0));
    forked = true;
    ctx->stream = ctx->aux_stream;
    if (NB > 0) rc = dgc_bands_to_taps(ctx, taps_or_bands_dev, w_dev, (int32_t)nFB, NB, NT, d_taps);
    if (rc == DGC_OK && !serial_fir) {
      dgc_fir_params fp = s->fir;
      fp.accumulate = 0;
      rc = dgc_fir_noise(ctx, &fp, noise_dev, d_taps, noise_gain_dev, d_noise);
    }
    cudaError_t e = cudaEventRecord(ctx->join_ev, ctx->aux_stream);
    ctx->stream = main_stream;
    if (rc == DGC_OK && e != cudaSuccess) rc = dgc_fail(ctx, DGC_ERR_CUDA, "event record: %s", cudaGetErrorString(e));
  }
  // the harmonic branch goes onto the caller's stream BEFORE that stream is told to wait for the noise branch
  if (rc == DGC_OK) {
    dgc_harmonic_params hp = s->harm;
    hp.accumulate = 0;
    rc = dgc_harmonic_render(ctx, &hp, f0_dev, uv_dev, amps_dev, gain_dev, nullptr, d_harm);
  }
  // join, whatever happened above: nothing of this call is left running beside the caller's stream
  if (forked) cudaStreamWaitEvent(main_stream, ctx->join_ev, 0);
  if (rc != DGC_OK) return rc;
  if (serial_fir) {
    dgc_fir_params fp = s->fir;
    fp.accumulate = 1;
    rc = dgc_fir_noise(ctx, &fp, noise_dev, d_taps, noise_gain_dev, d_harm);
    if (rc != DGC_OK) return rc;
  }
  if (ev_target) DGC_CUDA(ctx, cudaStreamWaitEvent(main_stream, ev_target, 0));
  if (audio_dev) {
    if (noise && !serial_fir) {
      add2_kernel<<<dgc_div_up((int64_t)nBT, 256), 256, 0, ctx->stream>>>(d_harm, d_noise, nBT, audio_dev);
      DGC_LAUNCHED(ctx, "add_branches");
    } else {
      DGC_CUDA(ctx, cudaMemcpyAsync(audio_dev, d_harm, nBT * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    }
    return dgc_mss_loss_fwd_sum(ctx, &s->mss, audio_dev, nullptr, target_dev, nullptr, loss_dev);
  }
  // Sum the branches in place first, then the plain loss kernel: measured 0.349 ms per step against 0.360 ms
  // with the loss kernel adding the two signals as it loads them (DGC_HN_SUM=fused selects that variant).
  static const bool add_first = [] {
    const char *e = getenv("DGC_HN_SUM");
    return !(e && strcmp(e, "fused") == 0);
  }();
  if (serial_fir) return dgc_mss_loss_fwd_sum(ctx, &s->mss, d_harm, nullptr, target_dev, nullptr, loss_dev);
  if (add_first && noise) {
    add2_kernel<<<dgc_div_up((int64_t)nBT, 256), 256, 0, ctx->stream>>>(d_harm, d_noise, nBT, d_harm);
    DGC_LAUNCHED(ctx, "add_branches");
    return dgc_mss_loss_fwd_sum(ctx, &s->mss, d_harm, nullptr, target_dev, nullptr, loss_dev);
  }
  return dgc_mss_loss_fwd_sum(ctx, &s->mss, d_harm, d_noise, target_dev, nullptr, loss_dev);
}

DGC_EXPORT int32_t dgc_hn_forward_loss(dgc_ctx *ctx, const dgc_hn_step *s, const float *f0_dev, const float *uv_dev,
                                       const float *amps_dev, const float *gain_dev, const float *noise_gain_dev,
                                       const float *taps_or_bands_dev, const float *w_dev, const float *noise_dev,
                                       const float *target_dev, float *work_dev, double *loss_dev, float *audio_dev) {
  return hn_forward_loss_impl(ctx, s, f0_dev, uv_dev, amps_dev, gain_dev, noise_gain_dev, taps_or_bands_dev, w_dev,
                              noise_dev, target_dev, work_dev, loss_dev, audio_dev, nullptr, nullptr);
}

// slot < 0: the blocking call (one staging area, returns after the loss has arrived).
// slot 0 / 1: one of two steps in flight -- inputs go to the slot's own staging area, so the upload of the next
// step crosses PCIe while this step computes; nothing is waited for here (dgc_hn_forward_loss_host_wait does).
static int32_t hn_host_enqueue(dgc_ctx *ctx, const dgc_hn_step *s, const float *f0_host, const float *uv_host,
                               const float *amps_host, const float *gain_host, const float *noise_gain_host,
                               const float *taps_or_bands_host, const float *w_host, const float *noise_host,
                               const float *target_host, double *loss_host, float *audio_host, int slot) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, s && f0_host && uv_host && amps_host && gain_host && loss_host, "null pointer");
  DGC_REQUIRE(ctx, target_host || s->target_dev, "the target must be given in host memory or as a resident device buffer");
  const int B = s->harm.B, T = s->harm.T, K = s->harm.K, F = s->harm.F;
  DGC_REQUIRE(ctx, B > 0 && T > 0 && K > 0 && F > 0, "size out of range");
  const int NT = s->fir.taps, NB = s->nbands;
  const bool noise = NT > 0;
  if (noise) {
    DGC_REQUIRE(ctx, noise_gain_host && taps_or_bands_host && (noise_host || s->noise_seed), "noise branch needs its inputs");
    DGC_REQUIRE(ctx, s->fir.B == B && s->fir.T == T && s->fir.F == F, "fir shape differs from harmonic shape");
    DGC_REQUIRE(ctx, NB == 0 || w_host, "band synthesis needs the matrix W");
  }
  DGC_REQUIRE(ctx, s->mss.B == B && s->mss.T == T, "loss shape differs from harmonic shape");
  const bool gen_noise = noise && !noise_host;          // generated on the device from s->noise_seed
  const bool resident_target = s->target_dev != nullptr;
  const uint64_t nFB = (uint64_t)F * B, nBT = (uint64_t)B * T;
  const uint64_t n_tab = noise ? nFB * (NB > 0 ? NB : NT) : 0;
  const uint64_t n_w = (noise && NB > 0) ? (uint64_t)NT * NB : 0;
  // host -> device inputs, in one contiguous pinned block
  const uint64_t in_floats = 3 * nFB + nFB * K + (noise ? nFB + n_tab + n_w + nBT : 0) + nBT;
  const uint64_t dev_extra = nBT /*audio*/ + dgc_hn_forward_loss_work_floats(s) + 64 * 16;
  const bool piped = slot >= 0;
  if (!piped)
    DGC_REQUIRE(ctx, !ctx->pipe_pending[0] && !ctx->pipe_pending[1],
                "steps submitted with dgc_hn_forward_loss_host_submit are still in flight: wait for them first");
  int32_t rc = ensure_stage(ctx, (piped ? 0 : in_floats) + dev_extra + 64 * 16);
  if (rc != DGC_OK) return rc;

  if (!ctx->copy_stream) {
    DGC_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
    for (auto &e : ctx->copy_ev) DGC_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  }
  cudaEvent_t *ev = ctx->copy_ev;
  if (piped) {
    const uint64_t need = in_floats + 64 * 16;
    if (ctx->pipe_in_floats[slot] < need) {
      if (ctx->pipe_in[slot]) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamSynchronize(ctx->copy_stream);
        cudaFree(ctx->pipe_in[slot]);
        ctx->buffer_generation++;
        ctx->pipe_in[slot] = nullptr;
        ctx->pipe_in_floats[slot] = 0;
      }
      DGC_CUDA(ctx, cudaMalloc(&ctx->pipe_in[slot], need * sizeof(float)));
      ctx->pipe_in_floats[slot] = need;
    }
    if (!ctx->pipe_done[slot]) {
      DGC_CUDA(ctx, cudaEventCreateWithFlags(&ctx->pipe_done[slot], cudaEventDisableTiming));
      for (auto &e : ctx->pipe_ev[slot]) DGC_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    ev = ctx->pipe_ev[slot];
    // the slot's previous step may still read its staging area: the new upload waits for that step's end
    if (ctx->pipe_pending[slot])
      return dgc_fail(ctx, DGC_ERR_INVALID, "slot %d still holds a step: call dgc_hn_forward_loss_host_wait first", slot);
    if (ctx->pipe_used[slot]) DGC_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->pipe_done[slot], 0));
  }
  // Blocking form: every earlier call ended with a stream synchronisation, so no kernel still reads the staging
  // area; work the caller queued on the context stream before this call does not touch it either.
  Carver dc(piped ? ctx->pipe_in[slot] : ctx->stage_dev);
  cudaError_t cp_err = cudaSuccess;
  static const bool inline_upload = [] {
    const char *e = getenv("DGC_UPLOAD");
    return e && strcmp(e, "inline") == 0;
  }();
  cudaStream_t up = inline_upload ? ctx->stream : ctx->copy_stream;
  auto put = [&](const float *src, uint64_t n) -> float * {
    float *d = dc.take(n);
    cudaError_t e = cudaMemcpyAsync(d, src, n * sizeof(float), cudaMemcpyHostToDevice, up);
    if (e != cudaSuccess && cp_err == cudaSuccess) cp_err = e;
    return d;
  };
  auto mark = [&](int i) {
    cudaError_t e = cudaEventRecord(ev[i], up);
    if (e != cudaSuccess && cp_err == cudaSuccess) cp_err = e;
  };
  // group 0: harmonic controls; group 1: noise branch; group 2: target
  float *d_f0 = put(f0_host, nFB), *d_uv = put(uv_host, nFB), *d_gain = put(gain_host, nFB);
  float *d_amps = put(amps_host, nFB * K);
  mark(0);
  float *d_ng = nullptr, *d_tab = nullptr, *d_w = nullptr, *d_noise = nullptr;
  if (noise) {
    d_ng = put(noise_gain_host, nFB);
    d_tab = put(taps_or_bands_host, n_tab);
    if (NB > 0) d_w = put(w_host, n_w);
    d_noise = gen_noise ? dc.take(nBT) : put(noise_host, nBT);
  }
  mark(1);
  float *d_target = resident_target ? const_cast<float *>(s->target_dev) : put(target_host, nBT);
  mark(2);
  if (cp_err != cudaSuccess) {
    cudaStreamSynchronize(ctx->copy_stream);
    return dgc_fail(ctx, DGC_ERR_CUDA, "input upload: %s", cudaGetErrorString(cp_err));
  }
  // from here on every exit path drains the upload stream before returning (the caller may reuse or free
  // its buffers as soon as this function returns)
  auto bail = [&](int32_t code) {
    cudaStreamSynchronize(ctx->copy_stream);
    return code;
  };
  // device work area of the two-branch step, and (only when the caller wants the audio back) the summed signal
  dgc_hn_step st = *s;
  // (two steps in flight share ONE work area: their kernels run one after the other on the context stream)
  Carver wc(ctx->stage_dev);
  Carver &work_carver = piped ? wc : dc;
  float *d_work = work_carver.take(dgc_hn_forward_loss_work_floats(&st));
  float *d_audio = audio_host ? work_carver.take(nBT) : nullptr;
  // the harmonic branch only needs group 0; the noise branch and the loss wait for their own uploads inside
  if (cudaStreamWaitEvent(ctx->stream, ev[0], 0) != cudaSuccess) return bail(dgc_fail(ctx, DGC_ERR_CUDA, "event wait"));
  if (gen_noise) {   // on the context stream, before the step forks its noise branch off it
    rc = dgc_noise_fill(ctx, s->noise_seed, s->noise_mode, B, T, s->noise_sigma, d_noise);
    if (rc != DGC_OK) return bail(rc);
  }
  double *loss_dev = ctx->loss_accum + (piped ? 1 + slot : 0);
  rc = hn_forward_loss_impl(ctx, &st, d_f0, d_uv, d_amps, d_gain, d_ng, d_tab, d_w, d_noise, d_target, d_work, loss_dev,
                            d_audio, inline_upload ? nullptr : ev[1], inline_upload ? nullptr : ev[2]);
  if (rc != DGC_OK) return bail(rc);
  DGC_CUDA(ctx, cudaMemcpyAsync(loss_host, loss_dev, sizeof(double), cudaMemcpyDeviceToHost, ctx->stream));
  if (audio_host)
    DGC_CUDA(ctx, cudaMemcpyAsync(audio_host, d_audio, nBT * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  if (!piped) return dgc_sync(ctx, 0);
  DGC_CUDA(ctx, cudaEventRecord(ctx->pipe_done[slot], ctx->stream));
  ctx->pipe_used[slot] = true;
  ctx->pipe_pending[slot] = true;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_hn_forward_loss_host(dgc_ctx *ctx, const dgc_hn_step *s, const float *f0_host,
                                            const float *uv_host, const float *amps_host, const float *gain_host,
                                            const float *noise_gain_host, const float *taps_or_bands_host,
                                            const float *w_host, const float *noise_host, const float *target_host,
                                            double *loss_host, float *audio_host) {
  return hn_host_enqueue(ctx, s, f0_host, uv_host, amps_host, gain_host, noise_gain_host, taps_or_bands_host, w_host,
                         noise_host, target_host, loss_host, audio_host, -1);
}

DGC_EXPORT int32_t dgc_hn_forward_loss_host_submit(dgc_ctx *ctx, const dgc_hn_step *s, const float *f0_host,
                                                   const float *uv_host, const float *amps_host,
                                                   const float *gain_host, const float *noise_gain_host,
                                                   const float *taps_or_bands_host, const float *w_host,
                                                   const float *noise_host, const float *target_host, int32_t slot,
                                                   double *loss_host, float *audio_host) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, slot == 0 || slot == 1, "slot must be 0 or 1");
  return hn_host_enqueue(ctx, s, f0_host, uv_host, amps_host, gain_host, noise_gain_host, taps_or_bands_host, w_host,
                         noise_host, target_host, loss_host, audio_host, slot);
}

DGC_EXPORT int32_t dgc_hn_forward_loss_host_wait(dgc_ctx *ctx, int32_t slot) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, slot == 0 || slot == 1, "slot must be 0 or 1");
  DGC_REQUIRE(ctx, ctx->pipe_pending[slot], "no step was submitted on this slot");
  ctx->pipe_pending[slot] = false;
  DGC_CUDA(ctx, cudaEventSynchronize(ctx->pipe_done[slot]));
  return DGC_OK;
}
