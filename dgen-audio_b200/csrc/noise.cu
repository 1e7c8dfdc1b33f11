// Signal.noise() on the device: the reference's xorshift32 generator (13, 17, 5; state bit-stored in a float
// cell, a zero state reseeded to 1, value = state / 2^32 in (0, 1); Sources/DGen/Renderer/CRenderer.swift:660-695),
// frame-parallel.
//
// The generator is a linear map M over GF(2)^32, so the state n steps ahead is M^n s: a thread that produces the
// values of one run of RUN consecutive frames first jumps to the run's start with the precomputed matrices
// M^(RUN 2^k) (one matrix-vector product per set bit of the run index, 32 conditional xors each) and then steps.
// Two forms:
//   DGC_NOISE_STREAM    the reference stream itself, bit for bit: out[b][n] = value n of the one stream started from
//                       `seed`, the same for every voice -- what `Signal.noise().buffer(size:).expand([B, size])`
//                       feeds the batched synthesiser (Examples/HarmonicE2E/Synth.swift:97-98);
//   DGC_NOISE_GAUSSIAN  white N(0, sigma) per voice for the synthetic harmonic+noise workload: voice b runs its own
//                       stream from a state hashed from (seed, b); frame n takes values 2n and 2n + 1 of it through
//                       Box-Muller, sigma sqrt(-2 ln u1) cos(2 pi u2).
#include "common.cuh"

#include <mutex>

namespace {

constexpr int RUN = 64;          // frames per thread
constexpr int JUMPS = 26;        // M^(RUN 2^k), k < JUMPS: streams of up to RUN * 2^26 values
__constant__ uint32_t c_jump[JUMPS][32];        // column i = image of bit i
__constant__ uint32_t c_jump2[JUMPS][32];       // the same for runs of 2 RUN steps (two values per frame)

__host__ __device__ inline uint32_t xs_step(uint32_t s) {
  s ^= s << 13;
  s ^= s >> 17;
  s ^= s << 5;
  return s;
}

__device__ __forceinline__ uint32_t apply(const uint32_t (*cols)[32], int k, uint32_t s) {
  uint32_t r = 0u;
#pragma unroll
  for (int i = 0; i < 32; ++i) r ^= (s >> i) & 1u ? cols[k][i] : 0u;
  return r;
}

template <bool PAIRS>
__device__ __forceinline__ uint32_t jump_to_run(uint32_t s, unsigned run) {
  for (int k = 0; k < JUMPS && (run >> k); ++k)
    if ((run >> k) & 1u) s = apply(PAIRS ? c_jump2 : c_jump, k, s);
  return s;
}

// splitmix-style hash of (seed, voice) to a non-zero stream state
__device__ __forceinline__ uint32_t voice_state(uint32_t seed, uint32_t b) {
  uint32_t z = seed + 0x9E3779B9u * (b + 1u);
  z = (z ^ (z >> 16)) * 0x85EBCA6Bu;
  z = (z ^ (z >> 13)) * 0xC2B2AE35u;
  z ^= z >> 16;
  return z ? z : 1u;
}

__global__ void noise_stream_kernel(uint32_t seed, int B, int T, float *__restrict__ out) {
  const unsigned run = blockIdx.x * blockDim.x + threadIdx.x;
  const int n0 = (int)run * RUN;
  if (n0 >= T) return;
  uint32_t s = jump_to_run<false>(seed ? seed : 1u, run);
  float v[RUN];
  const int n1 = min(T, n0 + RUN);
  for (int n = n0; n < n1; ++n) {
    s = xs_step(s);
    v[n - n0] = (float)s / 4294967296.0f;
  }
  for (int b = 0; b < B; ++b)
    for (int n = n0; n < n1; ++n) out[(size_t)b * T + n] = v[n - n0];
}

// One block = 64 threads = 64 runs = 4096 consecutive frames of one voice.  A thread's run is 256 contiguous bytes,
// so storing from the registers would make every store instruction touch 32 different 256-byte stretches; the runs
// go through a shared-memory tile instead (rows padded to 65 floats) and leave as full 128-byte row segments.
__global__ void __launch_bounds__(64) noise_gaussian_kernel(uint32_t seed, int B, int T, float sigma,
                                                             float *__restrict__ out) {
  __shared__ float tile[64][RUN + 1];
  const unsigned run = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y, n0 = (int)run * RUN;
  if (n0 < T) {
    uint32_t s = jump_to_run<true>(voice_state(seed, (uint32_t)b), run);
#pragma unroll 4
    for (int u = 0; u < RUN; ++u) {
      s = xs_step(s);
      const float u1 = (float)s / 4294967296.0f;
      s = xs_step(s);
      const float u2 = (float)s / 4294967296.0f;
      // u1 in (0, 1]: (float)s can round up to 2^32; log(1) = 0 is fine, log(0) cannot happen (s != 0)
      tile[threadIdx.x][u] = sigma * sqrtf(-2.0f * __logf(u1)) * __cosf(6.283185307179586f * u2);
    }
  }
  __syncthreads();
  const int base = (int)(blockIdx.x * blockDim.x) * RUN;
  float *o = out + (size_t)b * T;
  for (int i = threadIdx.x; i < 64 * RUN; i += 64) {
    const int n = base + i;
    if (n < T) o[n] = tile[i / RUN][i % RUN];
  }
}

// host: columns of M^(steps 2^k)
void build_jumps(int steps, uint32_t (*dst)[32]) {
  uint32_t m[32];
  for (int i = 0; i < 32; ++i) m[i] = xs_step(1u << i);          // M
  auto mul = [](const uint32_t *a, const uint32_t *b, uint32_t *c) {   // c = a b (apply b, then a)
    for (int i = 0; i < 32; ++i) {
      uint32_t col = b[i], r = 0u;
      for (int j = 0; j < 32; ++j)
        if ((col >> j) & 1u) r ^= a[j];
      c[i] = r;
    }
  };
  // M^steps by repeated squaring
  uint32_t p[32], acc[32], t[32];
  for (int i = 0; i < 32; ++i) {
    p[i] = m[i];
    acc[i] = 1u << i;
  }
  for (int e = steps; e; e >>= 1) {
    if (e & 1) {
      mul(p, acc, t);
      memcpy(acc, t, sizeof(t));
    }
    mul(p, p, t);
    memcpy(p, t, sizeof(t));
  }
  for (int k = 0; k < JUMPS; ++k) {
    memcpy(dst[k], acc, sizeof(acc));
    mul(acc, acc, t);
    memcpy(acc, t, sizeof(t));
  }
}

int32_t ensure_tables(dgc_ctx *ctx) {
  // per device: __constant__ memory belongs to the device's copy of the module
  static std::mutex mu;
  static bool done[64] = {false};
  std::lock_guard<std::mutex> lock(mu);
  if (ctx->device < 0 || ctx->device >= 64) return dgc_fail(ctx, DGC_ERR_INVALID, "noise: device index out of range");
  if (done[ctx->device]) return DGC_OK;
  static uint32_t j1[JUMPS][32], j2[JUMPS][32];
  build_jumps(RUN, j1);
  build_jumps(2 * RUN, j2);
  DGC_CUDA(ctx, cudaMemcpyToSymbol(c_jump, j1, sizeof(j1)));
  DGC_CUDA(ctx, cudaMemcpyToSymbol(c_jump2, j2, sizeof(j2)));
  done[ctx->device] = true;
  return DGC_OK;
}

}  // namespace

DGC_EXPORT int32_t dgc_noise_fill(dgc_ctx *ctx, uint32_t seed, int32_t mode, int32_t B, int32_t T, float sigma,
                                  float *out_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, out_dev, "null pointer");
  DGC_REQUIRE(ctx, B > 0 && B <= 65535 && T > 0, "size out of range");
  DGC_REQUIRE(ctx, mode == DGC_NOISE_STREAM || mode == DGC_NOISE_GAUSSIAN, "mode must be DGC_NOISE_STREAM or DGC_NOISE_GAUSSIAN");
  int32_t rc = ensure_tables(ctx);
  if (rc != DGC_OK) return rc;
  const int runs = dgc_div_up(T, RUN);
  if (mode == DGC_NOISE_STREAM) {
    noise_stream_kernel<<<dgc_div_up(runs, 64), 64, 0, ctx->stream>>>(seed, B, T, out_dev);
  } else {
    noise_gaussian_kernel<<<dim3(dgc_div_up(runs, 64), B), 64, 0, ctx->stream>>>(seed, B, T, sigma, out_dev);
  }
  DGC_LAUNCHED(ctx, "noise_fill");
  return DGC_OK;
}
