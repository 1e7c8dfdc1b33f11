// Context, arena, tables, timing: the plumbing every entry point of libdgen_cuda shares.
#include <math.h>
#include <stdarg.h>

#include <chrono>
#include <thread>
#include <vector>

#include "common.cuh"
#include "tma.cuh"

int32_t dgc_fail(dgc_ctx *ctx, int32_t code, const char *fmt, ...) {
  if (ctx) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
    va_end(ap);
  }
  return code;
}

int32_t dgc_check_launch(dgc_ctx *ctx, const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return dgc_fail(ctx, DGC_ERR_CUDA, "launch %s: %s", what, cudaGetErrorString(e));
  return DGC_OK;
}

float *dgc_ctx_scratch(dgc_ctx *ctx, uint64_t nfloats) {
  if (nfloats <= ctx->scratch_floats) return ctx->scratch;
  // the old buffer may still be in use by enqueued work: free it only after the stream drains
  if (ctx->scratch) {
    cudaStreamSynchronize(ctx->stream);
    cudaFree(ctx->scratch);
    ctx->scratch = nullptr;
    ctx->scratch_floats = 0;
    ctx->buffer_generation++;
  }
  float *p = nullptr;
  cudaError_t e = cudaMalloc(&p, nfloats * sizeof(float));
  if (e != cudaSuccess) {
    dgc_fail(ctx, DGC_ERR_OOM, "scratch of %llu floats: %s", (unsigned long long)nfloats, cudaGetErrorString(e));
    return nullptr;
  }
  ctx->scratch = p;
  ctx->scratch_floats = nfloats;
  return p;
}

template <typename T>
static T *upload_table(dgc_ctx *ctx, const std::vector<T> &h) {
  T *d = nullptr;
  if (cudaMalloc(&d, h.size() * sizeof(T)) != cudaSuccess) {
    dgc_fail(ctx, DGC_ERR_OOM, "table allocation failed");
    return nullptr;
  }
  // tables are tiny and built once: a synchronous copy keeps their lifetime simple
  if (cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) {
    dgc_fail(ctx, DGC_ERR_CUDA, "table upload failed");
    cudaFree(d);
    return nullptr;
  }
  return d;
}

// Symmetric Hann evaluated in double and rounded to float, as the reference builds its static
// window tensor for the spectral loss (Sources/DGen/HigherOps.swift:72-76).
const float *dgc_ctx_hann_sym(dgc_ctx *ctx, int N) {
  auto it = ctx->hann_sym.find(N);
  if (it != ctx->hann_sym.end()) return it->second;
  std::vector<float> h(N);
  for (int i = 0; i < N; ++i) h[i] = (float)(0.5 * (1.0 - cos(2.0 * M_PI * (double)i / (double)(N - 1))));
  float *d = upload_table(ctx, h);
  if (d) ctx->hann_sym[N] = d;
  return d;
}

// hann(n) of the public API: periodic, evaluated in single precision with Swift's Float.pi
// (pi rounded toward zero), Sources/DGenLazy/SpectralTensorOps.swift:42-49.
const float *dgc_ctx_hann_per(dgc_ctx *ctx, int N) {
  auto it = ctx->hann_per.find(N);
  if (it != ctx->hann_per.end()) return it->second;
  std::vector<float> h(N);
  const float swift_pi = 3.1415925025939941f;
  float scale = 2.0f * swift_pi / (float)N;
  for (int i = 0; i < N; ++i) h[i] = 0.5f - 0.5f * cosf(scale * (float)i);
  float *d = upload_table(ctx, h);
  if (d) ctx->hann_per[N] = d;
  return d;
}

// Frame ranges per control row, derived once per (F, T) from the cached control clock: the clock is
// data independent, so which frames interpolate from row r is a static table (like a window).
const int *dgc_ctx_row_ranges(dgc_ctx *ctx, int F, int T) {
  auto key = std::make_pair(F, T);
  auto it = ctx->row_ranges.find(key);
  if (it != ctx->row_ranges.end()) return it->second;
  const float *play_dev = nullptr;
  if (dgc_playhead(ctx, F, T, &play_dev) != DGC_OK) return nullptr;
  std::vector<float> play(T);
  if (cudaStreamSynchronize(ctx->stream) != cudaSuccess ||
      cudaMemcpy(play.data(), play_dev, (size_t)T * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) {
    dgc_fail(ctx, DGC_ERR_CUDA, "row_ranges: reading the control clock failed");
    return nullptr;
  }
  std::vector<int> tab((size_t)F * 4, 0);
  std::vector<int> runs(F, 0);
  int n = 0;
  while (n < T) {
    float w = fmodf(play[n], (float)F);
    if (w < 0) w += (float)F;
    int lo = (int)floorf(w), e = n + 1;
    while (e < T) {
      float w2 = fmodf(play[e], (float)F);
      if (w2 < 0) w2 += (float)F;
      if ((int)floorf(w2) != lo) break;
      ++e;
    }
    if (lo < 0 || lo >= F || runs[lo] >= 2) {
      dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "row_ranges: control row %d is visited in more than two runs", lo);
      return nullptr;
    }
    tab[(size_t)lo * 4 + 2 * runs[lo]] = n;
    tab[(size_t)lo * 4 + 2 * runs[lo] + 1] = e;
    runs[lo]++;
    n = e;
  }
  int *d = upload_table(ctx, tab);
  if (d) ctx->row_ranges[key] = d;
  return d;
}

const float2 *dgc_ctx_twiddles(dgc_ctx *ctx, int N) {
  auto it = ctx->twiddles.find(N);
  if (it != ctx->twiddles.end()) return it->second;
  std::vector<float2> h(N);
  for (int m = 0; m < N; ++m) {
    double a = -2.0 * M_PI * (double)m / (double)N;
    h[m] = make_float2((float)cos(a), (float)sin(a));
  }
  float2 *d = upload_table(ctx, h);
  if (d) ctx->twiddles[N] = d;
  return d;
}

DGC_EXPORT int32_t dgc_abi_version(void) { return DGC_ABI_VERSION; }

DGC_EXPORT int32_t dgc_ctx_create(int32_t device, dgc_ctx **out) {
  if (!out) return DGC_ERR_INVALID;
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return DGC_ERR_CUDA;
  if (cudaSetDevice(device) != cudaSuccess) return DGC_ERR_CUDA;
  dgc_ctx *c = new dgc_ctx();
  c->device = device;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) c->sm_count = prop.multiProcessorCount;
  bool ok = cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) == cudaSuccess &&
            cudaEventCreate(&c->ev_begin) == cudaSuccess && cudaEventCreate(&c->ev_end) == cudaSuccess &&
            cudaEventCreateWithFlags(&c->ev_sync, cudaEventDisableTiming) == cudaSuccess &&
            cudaMalloc(&c->status_dev, 2 * sizeof(int32_t)) == cudaSuccess &&
            cudaMalloc(&c->loss_accum, 512 * sizeof(double)) == cudaSuccess &&
            cudaMemset(c->status_dev, 0, 2 * sizeof(int32_t)) == cudaSuccess;
  c->ticket_dev = reinterpret_cast<unsigned int *>(c->status_dev + 1);
  if (!ok) {
    dgc_ctx_destroy(c);
    return DGC_ERR_CUDA;
  }
  c->stream = c->own_stream;
  *out = c;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_ctx_destroy(dgc_ctx *c) {
  if (!c) return DGC_ERR_INVALID;
  cudaSetDevice(c->device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  for (auto &kv : c->playheads) cudaFree(kv.second);
  for (auto &kv : c->row_ranges) cudaFree(kv.second);
  for (auto &kv : c->row_tables) cudaFree(kv.second);
  for (auto &kv : c->hann_sym) cudaFree(kv.second);
  for (auto &kv : c->hann_per) cudaFree(kv.second);
  for (auto &kv : c->twiddles) cudaFree(kv.second);
  if (c->scratch) cudaFree(c->scratch);
  if (c->comm) dgc_comm_destroy(c);
  if (c->stage_dev) cudaFree(c->stage_dev);
  for (int i = 0; i < 2; ++i) {
    if (c->pipe_in[i]) cudaFree(c->pipe_in[i]);
    if (c->pipe_done[i]) cudaEventDestroy(c->pipe_done[i]);
    for (auto &e : c->pipe_ev[i])
      if (e) cudaEventDestroy(e);
  }
  for (auto &e : c->copy_ev)
    if (e) cudaEventDestroy(e);
  if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
  if (c->fork_ev) cudaEventDestroy(c->fork_ev);
  if (c->join_ev) cudaEventDestroy(c->join_ev);
  if (c->aux_stream) cudaStreamDestroy(c->aux_stream);
  if (c->wt_buf) cudaFree(c->wt_buf);
  if (c->dzt_buf) cudaFree(c->dzt_buf);
  if (c->status_dev) cudaFree(c->status_dev);
  if (c->loss_accum) cudaFree(c->loss_accum);
  if (c->ev_begin) cudaEventDestroy(c->ev_begin);
  if (c->ev_end) cudaEventDestroy(c->ev_end);
  if (c->ev_sync) cudaEventDestroy(c->ev_sync);
  if (c->own_stream) cudaStreamDestroy(c->own_stream);
  delete c;
  return DGC_OK;
}

DGC_EXPORT const char *dgc_last_error(dgc_ctx *ctx) { return ctx ? ctx->err : "null context"; }

DGC_EXPORT int32_t dgc_ctx_set_stream(dgc_ctx *ctx, void *s, int32_t external) {
  if (!ctx) return DGC_ERR_INVALID;
  ctx->stream = external ? (cudaStream_t)s : ctx->own_stream;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_sync(dgc_ctx *ctx, uint32_t timeout_ms) {
  if (!ctx) return DGC_ERR_INVALID;
  if (timeout_ms == 0) {
    DGC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  } else {
    DGC_CUDA(ctx, cudaEventRecord(ctx->ev_sync, ctx->stream));
    auto t0 = std::chrono::steady_clock::now();
    for (;;) {
      cudaError_t e = cudaEventQuery(ctx->ev_sync);
      if (e == cudaSuccess) break;
      if (e != cudaErrorNotReady) return dgc_fail(ctx, DGC_ERR_CUDA, "sync: %s", cudaGetErrorString(e));
      auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
      if (ms > (long long)timeout_ms) return dgc_fail(ctx, DGC_ERR_TIMEOUT, "sync: stream still busy after %u ms", timeout_ms);
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
  int32_t st = 0;
  DGC_CUDA(ctx, cudaMemcpy(&st, ctx->status_dev, sizeof(st), cudaMemcpyDeviceToHost));
  if (st != 0) {
    cudaMemset(ctx->status_dev, 0, sizeof(int32_t));
    return dgc_fail(ctx, DGC_ERR_DEVICE, "device status word = %d", st);
  }
  return DGC_OK;
}

// ---- self-test of the failure reporting: both calls are bounded by construction ------------------------------
namespace {
// waits on an mbarrier that nothing ever arrives on, with the library's bounded wait cut down to `polls`:
// the wait gives up, the kernel records status 201 (the code of an expired pipeline wait) and returns
__global__ void selftest_expired_wait_kernel(uint32_t polls, int32_t *status) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) dgtma::mbar_init(&bar, 1);
  __syncthreads();
  const uint32_t a = dgtma::smem_addr(&bar);
  bool done = false;
  for (uint32_t it = 0; it < polls && !done; ++it) {
    uint32_t d;
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t"
        "}\n"
        : "=r"(d)
        : "r"(a), "r"(0u)
        : "memory");
    done = d != 0;
  }
  if (!done && threadIdx.x == 0) atomicExch(status, 201);
}
// keeps one thread busy for about `us` microseconds of the global timer (capped by the caller)
__global__ void selftest_busy_kernel(unsigned long long us) {
  unsigned long long t0, t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  do {
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  } while (t - t0 < us * 1000ull);
}
}  // namespace

DGC_EXPORT int32_t dgc_selftest_expired_wait(dgc_ctx *ctx, uint32_t polls) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, polls >= 1 && polls <= (1u << 20), "polls must be in 1 .. 2^20");
  selftest_expired_wait_kernel<<<1, 32, 0, ctx->stream>>>(polls, ctx->status_dev);
  DGC_LAUNCHED(ctx, "selftest_expired_wait");
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_selftest_busy(dgc_ctx *ctx, uint32_t milliseconds) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, milliseconds >= 1 && milliseconds <= 500, "milliseconds must be in 1 .. 500");
  selftest_busy_kernel<<<1, 1, 0, ctx->stream>>>((unsigned long long)milliseconds * 1000ull);
  DGC_LAUNCHED(ctx, "selftest_busy");
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_profile_begin(dgc_ctx *ctx) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_CUDA(ctx, cudaEventRecord(ctx->ev_begin, ctx->stream));
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_profile_end(dgc_ctx *ctx, float *ms) {
  if (!ctx || !ms) return DGC_ERR_INVALID;
  DGC_CUDA(ctx, cudaEventRecord(ctx->ev_end, ctx->stream));
  DGC_CUDA(ctx, cudaEventSynchronize(ctx->ev_end));
  DGC_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev_begin, ctx->ev_end));
  return DGC_OK;
}

DGC_EXPORT int64_t dgc_launch_count(dgc_ctx *ctx) { return ctx ? ctx->launches : -1; }

DGC_EXPORT int32_t dgc_arena_create(dgc_ctx *ctx, uint64_t nfloats, dgc_arena **out) {
  if (!ctx || !out) return DGC_ERR_INVALID;
  *out = nullptr;
  // the reference arena is at least 1024 floats (Sources/DGen/Runtime.swift:732-744)
  if (nfloats < 1024) nfloats = 1024;
  float *p = nullptr;
  DGC_CUDA(ctx, cudaMalloc(&p, nfloats * sizeof(float)));
  dgc_arena *a = new dgc_arena{ctx, p, nfloats, true};
  *out = a;
  return dgc_arena_zero(a);
}

DGC_EXPORT int32_t dgc_arena_wrap(dgc_ctx *ctx, float *dev, uint64_t nfloats, dgc_arena **out) {
  if (!ctx || !out) return DGC_ERR_INVALID;
  *out = nullptr;
  DGC_REQUIRE(ctx, dev && nfloats > 0, "null memory or zero size");
  DGC_REQUIRE(ctx, (((uintptr_t)dev) & 255) == 0, "the memory must be 256-byte aligned");
  *out = new dgc_arena{ctx, dev, nfloats, false};
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_arena_destroy(dgc_arena *a) {
  if (!a) return DGC_ERR_INVALID;
  cudaStreamSynchronize(a->ctx->stream);
  if (a->owned) cudaFree(a->ptr);
  delete a;
  return DGC_OK;
}

DGC_EXPORT float *dgc_arena_ptr(dgc_arena *a) { return a ? a->ptr : nullptr; }
DGC_EXPORT uint64_t dgc_arena_size(dgc_arena *a) { return a ? a->n : 0; }

DGC_EXPORT int32_t dgc_arena_zero(dgc_arena *a) {
  if (!a) return DGC_ERR_INVALID;
  DGC_CUDA(a->ctx, cudaMemsetAsync(a->ptr, 0, a->n * sizeof(float), a->ctx->stream));
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_arena_upload(dgc_arena *a, uint64_t off, const float *src, uint64_t n) {
  if (!a || (!src && n)) return DGC_ERR_INVALID;
  if (off > a->n || n > a->n - off) return dgc_fail(a->ctx, DGC_ERR_INVALID, "arena_upload: range outside the arena");
  DGC_CUDA(a->ctx, cudaMemcpyAsync(a->ptr + off, src, n * sizeof(float), cudaMemcpyHostToDevice, a->ctx->stream));
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_arena_download(dgc_arena *a, uint64_t off, float *dst, uint64_t n) {
  if (!a || (!dst && n)) return DGC_ERR_INVALID;
  if (off > a->n || n > a->n - off) return dgc_fail(a->ctx, DGC_ERR_INVALID, "arena_download: range outside the arena");
  DGC_CUDA(a->ctx, cudaMemcpyAsync(dst, a->ptr + off, n * sizeof(float), cudaMemcpyDeviceToHost, a->ctx->stream));
  DGC_CUDA(a->ctx, cudaStreamSynchronize(a->ctx->stream));
  return DGC_OK;
}

// ---- output sanitiser ---------------------------------------------------------------------------
namespace {
__device__ __forceinline__ float sanitize_bits(float v) {
  return ((__float_as_uint(v) & 0x7f800000u) == 0x7f800000u) ? 0.0f : v;
}
// Pure streaming kernel (4 B in + 4 B out per element): 128-bit accesses over the aligned body, grid-stride,
// scalar head / tail when the two pointers share a misalignment, all-scalar when they do not.
// (in and out may be the same buffer: no restrict, every element is read before it is written by the same thread)
__global__ void __launch_bounds__(256) sanitize_kernel(const float *in, float *out,
                                                       uint64_t n, uint64_t head, int vec_ok) {
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (uint64_t)gridDim.x * blockDim.x;
  if (!vec_ok) {
    for (uint64_t i = tid; i < n; i += nth) out[i] = sanitize_bits(in[i]);
    return;
  }
  if (tid < head) out[tid] = sanitize_bits(in[tid]);
  const uint64_t nv = (n - head) >> 2;
  const float4 *iv = reinterpret_cast<const float4 *>(in + head);
  float4 *ov = reinterpret_cast<float4 *>(out + head);
  uint64_t i = tid;
  for (; i + nth < nv; i += 2 * nth) {  // two independent 128-bit loads in flight per thread
    float4 a = __ldcs(iv + i), b = __ldcs(iv + i + nth);
    a.x = sanitize_bits(a.x); a.y = sanitize_bits(a.y); a.z = sanitize_bits(a.z); a.w = sanitize_bits(a.w);
    b.x = sanitize_bits(b.x); b.y = sanitize_bits(b.y); b.z = sanitize_bits(b.z); b.w = sanitize_bits(b.w);
    __stcs(ov + i, a);
    __stcs(ov + i + nth, b);
  }
  if (i < nv) {
    float4 a = __ldcs(iv + i);
    a.x = sanitize_bits(a.x); a.y = sanitize_bits(a.y); a.z = sanitize_bits(a.z); a.w = sanitize_bits(a.w);
    __stcs(ov + i, a);
  }
  const uint64_t tail0 = head + (nv << 2);
  if (tail0 + tid < n) out[tail0 + tid] = sanitize_bits(in[tail0 + tid]);
}
}  // namespace

DGC_EXPORT int32_t dgc_sanitize(dgc_ctx *ctx, const float *in_dev, uint64_t n, float *out_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  if (n == 0) return DGC_OK;
  DGC_REQUIRE(ctx, in_dev && out_dev, "null pointer");
  DGC_REQUIRE(ctx, (((uintptr_t)in_dev | (uintptr_t)out_dev) & 3) == 0, "pointers must be 4-byte aligned");
  const int vec_ok = (((uintptr_t)in_dev ^ (uintptr_t)out_dev) & 15) == 0;
  uint64_t head = ((16 - ((uintptr_t)in_dev & 15)) & 15) >> 2;  // scalars before the first 16-byte boundary
  if (head > n) head = n;
  // 8 resident CTAs of 256 threads per SM; never more blocks than 128-bit items
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx->device);
  uint64_t want = dgc_div_up((int64_t)((n >> 2) + 1), 256);
  int grid = (int)(want < (uint64_t)sms * 8 ? want : (uint64_t)sms * 8);
  sanitize_kernel<<<grid, 256, 0, ctx->stream>>>(in_dev, out_dev, n, head, vec_ok);
  DGC_LAUNCHED(ctx, "sanitize");
  return DGC_OK;
}

// ---- sum over frames of per-frame tensors ----------------------------------------------------------------------
// The reference accumulates per-frame parameter gradients into the parameter's gradient cell frame by frame
// (tensorAccumulate / memoryAccumulate, Sources/DGen/Emit+State.swift:50-115) and reads the cells on the host
// (Sources/DGenLazy/Backward.swift:132-165).  Here the frames are summed in two fixed-order steps (segments of
// frames per element in double, then the segment sums), so the result does not depend on scheduling.
namespace {
constexpr int RF_SEG = 256;   // frames per segment

__global__ void reduce_frames_seg_kernel(const float *__restrict__ x, int64_t T, int64_t E, int NS,
                                         double *__restrict__ part /* [NS][E] */) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int sgm = blockIdx.y;
  if (e >= E) return;
  const int64_t n0 = (int64_t)sgm * RF_SEG, n1 = n0 + RF_SEG < T ? n0 + RF_SEG : T;
  double acc = 0.0;
  int64_t n = n0;
  for (; n + 8 <= n1; n += 8) {   // eight independent loads in flight
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __ldcs(x + (n + j) * E + e);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += (double)v[j];
  }
  for (; n < n1; ++n) acc += (double)x[n * E + e];
  part[(int64_t)sgm * E + e] = acc;
}

__global__ void reduce_frames_sum_kernel(const double *__restrict__ part, int64_t E, int NS, float scale, int accumulate,
                                         float *__restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  double acc = 0.0;
  for (int s = 0; s < NS; ++s) acc += part[(int64_t)s * E + e];
  const float r = (float)(acc * (double)scale);
  out[e] = accumulate ? out[e] + r : r;
}
}  // namespace

DGC_EXPORT int32_t dgc_reduce_frames(dgc_ctx *ctx, const float *x_dev, int64_t T, int64_t E, float scale,
                                     int32_t accumulate, float *out_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, x_dev && out_dev, "null pointer");
  DGC_REQUIRE(ctx, T > 0 && E > 0, "size out of range");
  const int64_t NS64 = (T + RF_SEG - 1) / RF_SEG;
  DGC_REQUIRE(ctx, NS64 <= 65535 && (E + 127) / 128 < 0x7fffffffLL, "size out of range");
  const int NS = (int)NS64;
  float *scr = dgc_ctx_scratch(ctx, 2ull * (uint64_t)NS * (uint64_t)E + 4);
  if (!scr) return DGC_ERR_OOM;
  double *part = reinterpret_cast<double *>(scr);
  reduce_frames_seg_kernel<<<dim3((unsigned)((E + 127) / 128), NS), 128, 0, ctx->stream>>>(x_dev, T, E, NS, part);
  DGC_LAUNCHED(ctx, "reduce_frames_segments");
  reduce_frames_sum_kernel<<<(unsigned)((E + 127) / 128), 128, 0, ctx->stream>>>(part, E, NS, scale, accumulate, out_dev);
  DGC_LAUNCHED(ctx, "reduce_frames_sum");
  return DGC_OK;
}
