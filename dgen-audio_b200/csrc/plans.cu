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
    ctx->stage_dev = nullptr;
    ctx->stage_floats = 0;
  }
  DGC_CUDA(ctx, cudaMalloc(&ctx->stage_dev, nfloats * sizeof(float)));
  ctx->stage_floats = nfloats;
  return DGC_OK;
}

}  // namespace

DGC_EXPORT int32_t dgc_hn_forward_loss_host(dgc_ctx *ctx, const dgc_hn_step *s, const float *f0_host,
                                            const float *uv_host, const float *amps_host, const float *gain_host,
                                            const float *noise_gain_host, const float *taps_or_bands_host,
                                            const float *w_host, const float *noise_host, const float *target_host,
                                            double *loss_host, float *audio_host) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, s && f0_host && uv_host && amps_host && gain_host && target_host && loss_host, "null pointer");
  const int B = s->harm.B, T = s->harm.T, K = s->harm.K, F = s->harm.F;
  DGC_REQUIRE(ctx, B > 0 && T > 0 && K > 0 && F > 0, "size out of range");
  const int NT = s->fir.taps, NB = s->nbands;
  const bool noise = NT > 0;
  if (noise) {
    DGC_REQUIRE(ctx, noise_gain_host && taps_or_bands_host && noise_host, "noise branch needs its inputs");
    DGC_REQUIRE(ctx, s->fir.B == B && s->fir.T == T && s->fir.F == F, "fir shape differs from harmonic shape");
    DGC_REQUIRE(ctx, NB == 0 || w_host, "band synthesis needs the matrix W");
  }
  DGC_REQUIRE(ctx, s->mss.B == B && s->mss.T == T, "loss shape differs from harmonic shape");
  const uint64_t nFB = (uint64_t)F * B, nBT = (uint64_t)B * T;
  const uint64_t n_tab = noise ? nFB * (NB > 0 ? NB : NT) : 0;
  const uint64_t n_w = (noise && NB > 0) ? (uint64_t)NT * NB : 0;
  // host -> device inputs, in one contiguous pinned block
  const uint64_t in_floats = 3 * nFB + nFB * K + (noise ? nFB + n_tab + n_w + nBT : 0) + nBT;
  const uint64_t dev_extra = nBT /*audio*/ + (noise && NB > 0 ? nFB * NT : 0) + 64 * 16;
  int32_t rc = ensure_stage(ctx, in_floats + dev_extra + 64 * 16);
  if (rc != DGC_OK) return rc;

  if (!ctx->copy_stream) {
    DGC_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
    for (auto &e : ctx->copy_ev) DGC_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  }
  // Every earlier call ended with a stream synchronisation, so no kernel still reads the staging area;
  // work the caller queued on the context stream before this call does not touch it either.
  Carver dc(ctx->stage_dev);
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
    cudaError_t e = cudaEventRecord(ctx->copy_ev[i], up);
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
    d_noise = put(noise_host, nBT);
  }
  mark(1);
  float *d_target = put(target_host, nBT);
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
  float *d_audio = dc.take(nBT);
  float *d_taps = d_tab;
  dgc_harmonic_params hp = s->harm;
  hp.accumulate = 0;
  if (cudaStreamWaitEvent(ctx->stream, ctx->copy_ev[0], 0) != cudaSuccess) return bail(dgc_fail(ctx, DGC_ERR_CUDA, "event wait"));
  rc = dgc_harmonic_render(ctx, &hp, d_f0, d_uv, d_amps, d_gain, nullptr, d_audio);
  if (rc != DGC_OK) return bail(rc);
  if (cudaStreamWaitEvent(ctx->stream, ctx->copy_ev[1], 0) != cudaSuccess) return bail(dgc_fail(ctx, DGC_ERR_CUDA, "event wait"));
  if (noise && NB > 0) {
    d_taps = dc.take(nFB * NT);
    rc = dgc_bands_to_taps(ctx, d_tab, d_w, (int32_t)nFB, NB, NT, d_taps);
    if (rc != DGC_OK) return bail(rc);
  }
  if (noise) {
    dgc_fir_params fp = s->fir;
    fp.accumulate = 1;
    rc = dgc_fir_noise(ctx, &fp, d_noise, d_taps, d_ng, d_audio);
    if (rc != DGC_OK) return bail(rc);
  }
  if (cudaStreamWaitEvent(ctx->stream, ctx->copy_ev[2], 0) != cudaSuccess) return bail(dgc_fail(ctx, DGC_ERR_CUDA, "event wait"));
  rc = dgc_mss_loss_fwd(ctx, &s->mss, d_audio, d_target, nullptr, ctx->loss_accum);
  if (rc != DGC_OK) return bail(rc);
  DGC_CUDA(ctx, cudaMemcpyAsync(loss_host, ctx->loss_accum, sizeof(double), cudaMemcpyDeviceToHost, ctx->stream));
  if (audio_host)
    DGC_CUDA(ctx, cudaMemcpyAsync(audio_host, d_audio, nBT * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  return dgc_sync(ctx, 0);
}
