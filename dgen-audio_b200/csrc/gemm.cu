// Controller layers and optimiser: dense fp32 matmul (+ bias, tanh), its backward, and Adam.
//
// The reference expresses a layer as mul + sumAxis over a broadcast [M,N,K] product on the C backend
// and as 8x8 simdgroup tiles on Metal (Sources/DGen/Tensor.swift:1195-1230, Sources/DGen/Emit+GEMM.swift);
// parameters live on the host and Adam is a per-element Swift loop (Sources/DGenLazy/Optimizers.swift:164-243).
// Here activations, weights, gradients and optimiser state stay in HBM.  The matmul runs on the
// tcgen05 tensor cores in 3xTF32 (tc_gemm.cuh: fp32-grade accuracy, which the gradient tolerance of the
// path -- 1e-3 relative against an fp64 evaluation -- needs; single-pass TF32 would not do), and a
// register-tiled SIMT kernel covers small shapes.
#include <stdlib.h>

#include "common.cuh"
#include "tc_gemm.cuh"

namespace {

// C[M][N] (+)= op(A) * op(B) with 128x128 block tiles, 8-deep k-slices, 8x8 register tiles per thread.
// TA: A is stored [K][M] (use A^T);  TB: B is stored [N][K] (use B^T).
constexpr int BM = 128, BN = 128, BK = 8, TM = 8, TN = 8;

// EPI 0: C = acc ; 1: C = acc + bias[n] ; 2: C = tanh(acc + bias[n])
template <bool TA, bool TB, int EPI>
__global__ void __launch_bounds__(256)
sgemm_kernel(const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ bias, int M, int N,
             int K, int k_per_split, float *__restrict__ C) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, each 8 x 8 outputs
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  // split-K: slice blockIdx.z of the reduction range goes to its own [M][N] slab of C
  const int k_begin = blockIdx.z * k_per_split;
  const int k_end = min(K, k_begin + k_per_split);
  C += (size_t)blockIdx.z * M * N;
  for (int k0 = k_begin; k0 < k_end; k0 += BK) {
    // stage A tile [BM][BK] and B tile [BK][BN]: 1024 elements each, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int idx = tid + e * 256;
      if (!TA) {  // A stored [M][K]: consecutive idx walk k fastest
        int m = idx / BK, k = idx % BK;
        int gm = m0 + m, gk = k0 + k;
        As[k][m] = (gm < M && gk < k_end) ? A[(size_t)gm * K + gk] : 0.0f;
      } else {    // A stored [K][M]: consecutive idx walk m fastest
        int k = idx / BM, m = idx % BM;
        int gm = m0 + m, gk = k0 + k;
        As[k][m] = (gm < M && gk < k_end) ? A[(size_t)gk * M + gm] : 0.0f;
      }
      if (!TB) {  // B stored [K][N]
        int k = idx / BN, n = idx % BN;
        int gn = n0 + n, gk = k0 + k;
        Bs[k][n] = (gn < N && gk < k_end) ? B[(size_t)gk * N + gn] : 0.0f;
      } else {    // B stored [N][K]
        int n = idx / BK, k = idx % BK;
        int gn = n0 + n, gk = k0 + k;
        Bs[k][n] = (gn < N && gk < k_end) ? B[(size_t)gn * K + gk] : 0.0f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; i += 4) {
        float4 v = *reinterpret_cast<const float4 *>(&As[k][ty * 4 + i * 16]);  // rows ty*4 + {0..3} + i*16... see below
        a[i] = v.x; a[i + 1] = v.y; a[i + 2] = v.z; a[i + 3] = v.w;
      }
#pragma unroll
      for (int j = 0; j < TN; j += 4) {
        float4 v = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4 + j * 16]);
        b[j] = v.x; b[j + 1] = v.y; b[j + 2] = v.z; b[j + 3] = v.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  // thread (ty, tx) owns rows m0 + ty*4 + {0..3} and m0 + 64 + ty*4 + {0..3}; same pattern for columns
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int gm = m0 + ty * 4 + (i & 3) + (i >> 2) * 64;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int gn = n0 + tx * 4 + (j & 3) + (j >> 2) * 64;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (EPI >= 1) v += bias[gn];
      if (EPI == 2) v = tanhf(v);
      C[(size_t)gm * N + gn] = v;
    }
  }
}

// C[m][n] = sum_z part[z][m][n], z ascending: fixed order, bit-reproducible
__global__ void splitk_reduce_kernel(const float *__restrict__ part, size_t mn, int splits, float *__restrict__ C) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= mn) return;
  float acc = 0.0f;
  for (int z = 0; z < splits; ++z) acc += part[(size_t)z * mn + i];
  C[i] = acc;
}

// true unless DGC_GEMM=simt is set in the environment (keeps the SIMT kernel reachable for comparison)
bool use_tensor_cores() {
  static int v = -1;
  if (v < 0) {
    const char *e = getenv("DGC_GEMM");
    v = (e && strcmp(e, "simt") == 0) ? 0 : 1;
  }
  return v == 1;
}

// true when C = A B^T of this shape runs on the persistent short-reduction tensor-core kernel: 32 <= K <= 72, at
// least one full block of 128 columns, A 16-byte aligned (its row tiles are fetched by bulk copies), no more column
// blocks than SMs.  DGC_GEMM_SMALLK=0 keeps such shapes on the general pipeline.
bool smallk_shape(const dgc_ctx *ctx, const float *A, int M, int N, int K) {
  static const bool on = [] {
    const char *e = getenv("DGC_GEMM_SMALLK");
    return !(e && atoi(e) == 0);
  }();
  if (!on || !use_tensor_cores() || (double)M * N * K < (double)(1 << 21) || K < 32 || K > dgtc::SK::KP_MAX ||
      N < dgtc::TBN || (((uintptr_t)A) & 15) != 0)
    return false;
  const int rem = N % dgtc::TBN;
  const int nblk = (rem > 0 && rem <= dgtc::SK::EXTRA_MAX) ? N / dgtc::TBN : dgc_div_up(N, dgtc::TBN);
  return nblk <= ctx->sm_count;
}

template <bool TA, bool TB, int EPI>
int32_t launch_sgemm(dgc_ctx *ctx, const float *A, const float *B, const float *bias, int M, int N, int K, float *C,
                     float *Ct = nullptr, bool *ct_written = nullptr) {
  if (ct_written) *ct_written = false;
  const bool tc = use_tensor_cores() && (double)M * N * K >= (double)(1 << 21) && K >= 32;
  static const int kk_bk = [] {   // DGC_GEMM_KK: 0 off; 16 (default) / 32: swizzled 16- / 32-wide k tiles; 17 / 33: the
                                  // same without swizzle; 256: 16-wide k tiles with 128 x 256 output tiles where N >= 256
    const char *e = getenv("DGC_GEMM_KK");
    return e ? atoi(e) : 16;
  }();
  // the asynchronous pipeline needs both operands contiguous along k, K a multiple of 4 and aligned rows
  const bool kk16 = tc && !TA && TB && kk_bk && (K & 3) == 0 && ((((uintptr_t)A) | ((uintptr_t)B)) & 15) == 0;
  // rows that are not 16-byte aligned (K % 4 != 0, e.g. 65 band magnitudes): the same pipeline with 4-byte copies
  const bool kk4 = tc && !TA && TB && kk_bk && !kk16 && EPI == 0;
  const bool kk = kk16 || kk4;
  // 128 x 256 tiles, one CTA per SM: 25 % less shared-memory traffic per flop, but prologue and epilogue are no
  // longer hidden by a second resident CTA, so they only pay where a CTA runs a long reduction -- the split-K
  // weight gradients (measured: training step 3.84 -> 3.78 ms; the forward layers get 4 % slower with them).
  // DGC_GEMM_KK=256 forces them wherever N >= 256.
  const bool long_reduction = EPI == 0 && K >= 2048 && dgc_div_up(N, dgtc::TBN) * dgc_div_up(M, dgtc::TBM) < ctx->sm_count;
  const bool wide = kk16 && N >= 256 && (kk_bk == 256 || (kk_bk == 16 && long_reduction));
  // short reductions (the band -> tap map): persistent CTAs that keep their block of B in shared memory
  if (!TA && TB && EPI == 0 && smallk_shape(ctx, A, M, N, K)) {
    const int rem = N % dgtc::TBN;
    const int n_extra = (rem > 0 && rem <= dgtc::SK::EXTRA_MAX) ? rem : 0;
    const int nblk = n_extra ? N / dgtc::TBN : dgc_div_up(N, dgtc::TBN);
    const int per = std::min(dgc_div_up(M, dgtc::TBM), ctx->sm_count / nblk);
    auto kern = dgtc::tc_gemm_smallk_kernel;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dgtc::SK::SMEM);
    if (e != cudaSuccess) return dgc_fail(ctx, DGC_ERR_CUDA, "tc_gemm smem opt-in: %s", cudaGetErrorString(e));
    ctx->gemm_paths[2]++;
    kern<<<nblk * per, dgtc::SK::THREADS_ALL, dgtc::SK::SMEM, ctx->stream>>>(A, B, M, N, K, nblk, n_extra, per, C,
                                                                             ctx->status_dev);
    return DGC_OK;
  }
  const int bm = tc ? dgtc::TBM : BM, bn = wide ? 256 : (tc ? dgtc::TBN : BN);
  const int tiles = dgc_div_up(N, bn) * dgc_div_up(M, bm);
  int splits = 1;
  if (EPI == 0 && tiles < ctx->sm_count && K >= 2048) {
    // few output tiles and a long reduction (weight gradients): split the reduction over blocks -- two resident
    // CTAs per SM for the narrow tiles, one (and never a second, nearly empty wave) for the wide ones
    splits = wide ? ctx->sm_count / tiles : (2 * ctx->sm_count + tiles - 1) / tiles;
    if (splits > K / 256) splits = K / 256;
    if (splits < 1) splits = 1;
  }
  int kps = K;
  float *dst = C;
  if (splits > 1) {
    kps = dgc_div_up(dgc_div_up(K, splits), 32) * 32;
    splits = dgc_div_up(K, kps);
    dst = dgc_ctx_scratch(ctx, (uint64_t)splits * M * N + 4);
    if (!dst) return DGC_ERR_OOM;
  }
  dim3 grid(dgc_div_up(N, bn), dgc_div_up(M, bm), splits);
  ctx->gemm_paths[(kk && (splits == 1 || kps % 32 == 0)) ? (wide ? 3 : 2) : (tc ? 1 : 0)]++;
  if (kk && (splits == 1 || kps % 32 == 0)) {
    // both operands contiguous along k: the cp.async pipeline
#define DGC_KK_LAUNCH(BKV, SWV)                                                                                      \
  do {                                                                                                              \
    auto kern = dgtc::tc_gemm_kk_kernel<EPI, BKV, SWV, dgtc::TBN>;                                                  \
    constexpr int SM = dgtc::KK<BKV, SWV, dgtc::TBN>::SMEM;                                                         \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM);                    \
    if (e != cudaSuccess) return dgc_fail(ctx, DGC_ERR_CUDA, "tc_gemm smem opt-in: %s", cudaGetErrorString(e));     \
    kern<<<grid, dgtc::KK_THREADS, SM, ctx->stream>>>(A, B, bias, M, N, K, kps, dst, splits == 1 ? Ct : nullptr,    \
                                                   ctx->status_dev);                                                \
  } while (0)
    if (kk4) {
      auto kern = dgtc::tc_gemm_kk_kernel<0, 16, true, dgtc::TBN, true>;
      constexpr int SM = dgtc::KK<16, true, dgtc::TBN>::SMEM;
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM);
      if (e != cudaSuccess) return dgc_fail(ctx, DGC_ERR_CUDA, "tc_gemm smem opt-in: %s", cudaGetErrorString(e));
      kern<<<grid, dgtc::KK_THREADS, SM, ctx->stream>>>(A, B, nullptr, M, N, K, kps, dst, nullptr, ctx->status_dev);
    } else if (wide) {
      auto kern = dgtc::tc_gemm_kk_kernel<EPI, 16, true, 256>;
      constexpr int SM = dgtc::KK<16, true, 256>::SMEM;
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM);
      if (e != cudaSuccess) return dgc_fail(ctx, DGC_ERR_CUDA, "tc_gemm smem opt-in: %s", cudaGetErrorString(e));
      kern<<<grid, dgtc::KK_THREADS, SM, ctx->stream>>>(A, B, bias, M, N, K, kps, dst, splits == 1 ? Ct : nullptr,
                                                         ctx->status_dev);
    } else if (kk_bk == 16 || kk_bk == 256) DGC_KK_LAUNCH(16, true);
    else if (kk_bk == 17) DGC_KK_LAUNCH(16, false);
    else if (kk_bk == 33) DGC_KK_LAUNCH(32, false);
    else DGC_KK_LAUNCH(32, true);
#undef DGC_KK_LAUNCH
    if (ct_written) *ct_written = Ct && splits == 1;
  } else if (tc) {
    // tensor-core kernel: operand A is K-major in memory when it is NOT transposed ([M][K]);
    // operand B is K-major in memory when it IS given transposed ([N][K])
    auto kern = dgtc::tc_gemm_kernel<!TA, TB, EPI>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dgtc::SMEM_BYTES);
    if (e != cudaSuccess) return dgc_fail(ctx, DGC_ERR_CUDA, "tc_gemm smem opt-in: %s", cudaGetErrorString(e));
    kern<<<grid, dgtc::THREADS, dgtc::SMEM_BYTES, ctx->stream>>>(A, B, bias, M, N, K, kps, dst, ctx->status_dev);
  } else {
    sgemm_kernel<TA, TB, EPI><<<grid, 256, 0, ctx->stream>>>(A, B, bias, M, N, K, kps, dst);
  }
  if (splits > 1) {
    ctx->launches++;
    size_t mn = (size_t)M * N;
    splitk_reduce_kernel<<<dgc_div_up((int64_t)mn, 256), 256, 0, ctx->stream>>>(dst, mn, splits, C);
  }
  return DGC_OK;
}

// out[c][r] = in[r][c] (small weight matrices only), 32 x 32 tiles through shared memory
__global__ void transpose_kernel(const float *__restrict__ in, int R, int Cc, float *__restrict__ out) {
  __shared__ float t[32][33];
  int c = blockIdx.x * 32 + threadIdx.x, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += 8)
    if (r0 + i < R && c < Cc) t[i][threadIdx.x] = in[(size_t)(r0 + i) * Cc + c];
  __syncthreads();
  int r = r0 + threadIdx.x, c0 = blockIdx.x * 32;
  for (int i = threadIdx.y; i < 32; i += 8)
    if (c0 + i < Cc && r < R) out[(size_t)(c0 + i) * R + r] = t[threadIdx.x][i];
}

// dZ = dC * act'(C) written twice: dZ[m][n] and the transposed copy dZt[n][m] (32 x 32 tiles through shared
// memory), so that the weight-gradient product can read both of its operands along the reduction index
__global__ void act_bwd_t_kernel(const float *__restrict__ dC, const float *__restrict__ Cv, int M, int N, int act,
                                 float *__restrict__ dZ, float *__restrict__ dZt) {
  __shared__ float t[32][33];
  const int n = blockIdx.x * 32 + threadIdx.x, m0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int m = m0 + i;
    float g = 0.0f;
    if (m < M && n < N) {
      const size_t idx = (size_t)m * N + n;
      g = dC[idx];
      if (act == 1) {
        const float c = Cv[idx];
        g *= (1.0f - c * c);
      }
      dZ[idx] = g;
    }
    t[i][threadIdx.x] = g;
  }
  __syncthreads();
  const int m = m0 + threadIdx.x, nb = blockIdx.x * 32;
  for (int i = threadIdx.y; i < 32; i += 8)
    if (nb + i < N && m < M) dZt[(size_t)(nb + i) * M + m] = t[threadIdx.x][i];
}

// dZ = dC * (1 - C^2) in place-compatible form (tanh'), or copy when act == 0
__global__ void act_bwd_kernel(const float *__restrict__ dC, const float *__restrict__ Cv, size_t n, int act,
                               float *__restrict__ dZ) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float g = dC[i];
  if (act == 1) {
    float c = Cv[i];
    g *= (1.0f - c * c);
  }
  dZ[i] = g;
}

// the same, four elements per thread (n a multiple of 4, 16-byte aligned buffers)
__global__ void act_bwd4_kernel(const float4 *__restrict__ dC, const float4 *__restrict__ Cv, size_t n4, int act,
                                float4 *__restrict__ dZ) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 g = dC[i];
  if (act == 1) {
    const float4 c = Cv[i];
    g.x *= (1.0f - c.x * c.x);
    g.y *= (1.0f - c.y * c.y);
    g.z *= (1.0f - c.z * c.z);
    g.w *= (1.0f - c.w * c.w);
  }
  dZ[i] = g;
}

// A layer with a handful of inputs (the controller's first layer: K = 2 features) is not a matmul but a streaming
// map: C[m][n] = act(sum_k A[m][k] W[k][n] + bias[n]).  One thread per four consecutive outputs of a row: the K
// inputs of the row are broadcast loads, W and the bias stay in L1, the store is 16 bytes.  Same operation order as
// the tile kernel (k ascending from zero, then the bias, then the library tanh).
template <int KK, int EPI>
__global__ void __launch_bounds__(256)
smallk_fwd_kernel(const float *__restrict__ A, const float *__restrict__ W, const float *__restrict__ bias, int M, int N,
                  float *__restrict__ C) {
  const int nq = N >> 2;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)M * nq) return;
  const int m = (int)(idx / nq), n = (int)(idx - (size_t)m * nq) * 4;
  float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int k = 0; k < KK; ++k) {
    const float a = __ldg(A + (size_t)m * KK + k);
    const float4 w = __ldg(reinterpret_cast<const float4 *>(W + (size_t)k * N + n));
    v[0] = fmaf(a, w.x, v[0]);
    v[1] = fmaf(a, w.y, v[1]);
    v[2] = fmaf(a, w.z, v[2]);
    v[3] = fmaf(a, w.w, v[3]);
  }
  if (EPI >= 1) {
    const float4 bq = __ldg(reinterpret_cast<const float4 *>(bias + n));
    v[0] += bq.x; v[1] += bq.y; v[2] += bq.z; v[3] += bq.w;
  }
  if (EPI == 2) {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = tanhf(v[j]);
  }
  *reinterpret_cast<float4 *>(C + (size_t)m * N + n) = make_float4(v[0], v[1], v[2], v[3]);
}

// Its backward: db[n] = sum_m dZ[m][n] and dW[k][n] = sum_m A[m][k] dZ[m][n] from ONE pass over dZ (a matmul
// with a 32000-long reduction and a 2 x 512 output reads dZ at a fraction of the memory rate).  Same two fixed-order
// stages as the bias gradient: block (32 columns x 1024 rows) -> part[chunk][1 + KK][n], then the chunks in order.
template <int KK>
__global__ void __launch_bounds__(256)
smallk_grad_kernel(const float *__restrict__ A, const float *__restrict__ dZ, int M, int N, float *__restrict__ part) {
  __shared__ float sh[KK + 1][8][33];
  __shared__ float as[1024 * KK];          // the chunk's rows of A: one coalesced read, then broadcast loads
  const int lane = threadIdx.x & 31, col = blockIdx.x * 32 + lane, rg = threadIdx.x >> 5;
  const int m_begin = blockIdx.y * 1024, m_end = min(M, m_begin + 1024);
  for (int i = threadIdx.x; i < (m_end - m_begin) * KK; i += 256) as[i] = A[(size_t)m_begin * KK + i];
  __syncthreads();
  float acc[KK + 1];
#pragma unroll
  for (int q = 0; q <= KK; ++q) acc[q] = 0.0f;
  if (col < N) {
#pragma unroll 4
    for (int m = m_begin + rg; m < m_end; m += 8) {
      const float d = dZ[(size_t)m * N + col];
      acc[0] += d;
#pragma unroll
      for (int k = 0; k < KK; ++k) acc[1 + k] = fmaf(as[(m - m_begin) * KK + k], d, acc[1 + k]);
    }
  }
#pragma unroll
  for (int q = 0; q <= KK; ++q) sh[q][rg][lane] = acc[q];
  __syncthreads();
  if (rg == 0 && col < N) {
#pragma unroll
    for (int q = 0; q <= KK; ++q) {
      float t = 0.0f;
#pragma unroll
      for (int r = 0; r < 8; ++r) t += sh[q][r][lane];
      part[((size_t)blockIdx.y * (KK + 1) + q) * N + col] = t;
    }
  }
}

// db (may be null) and dW from the chunk sums, chunks in index order
__global__ void smallk_grad_reduce_kernel(const float *__restrict__ part, int chunks, int KK, int N, float *__restrict__ db,
                                          float *__restrict__ dW) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (KK + 1) * N) return;
  const int q = i / N, col = i - q * N;
  float t = 0.0f;
  for (int c = 0; c < chunks; ++c) t += part[((size_t)c * (KK + 1) + q) * N + col];
  if (q == 0) {
    if (db) db[col] = t;
  } else
    dW[(size_t)(q - 1) * N + col] = t;
}

// db[n] = sum_m dZ[m][n].  Stage 1: block (32 columns x 1024 rows) sums its rows in a fixed order into
// part[chunk][n]; stage 2 adds the chunks in index order: bit-reproducible.
__global__ void __launch_bounds__(256)
bias_grad_kernel(const float *__restrict__ dZ, int M, int N, float *__restrict__ part) {
  __shared__ float sh[8][33];
  const int col = blockIdx.x * 32 + (threadIdx.x & 31), rg = threadIdx.x >> 5;
  const int m_begin = blockIdx.y * 1024, m_end = min(M, m_begin + 1024);
  float acc = 0.0f;
  if (col < N)
    for (int m = m_begin + rg; m < m_end; m += 8) acc += dZ[(size_t)m * N + col];
  sh[rg][threadIdx.x & 31] = acc;
  __syncthreads();
  if (rg == 0 && col < N) {
    float t = 0.0f;
#pragma unroll
    for (int r = 0; r < 8; ++r) t += sh[r][threadIdx.x & 31];
    part[(size_t)blockIdx.y * N + col] = t;
  }
}

__global__ void bias_grad_reduce_kernel(const float *__restrict__ part, int chunks, int N, float *__restrict__ db) {
  int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= N) return;
  float t = 0.0f;
  for (int c = 0; c < chunks; ++c) t += part[(size_t)c * N + col];
  db[col] = t;
}

__global__ void adam_kernel(float *__restrict__ theta, const float *__restrict__ g, float *__restrict__ m,
                            float *__restrict__ v, size_t n, float lr, float b1, float b2, float eps, float c1,
                            float c2) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  // operation order of Optimizers.swift:188-203
  float gi = g[i];
  float mi = __fadd_rn(__fmul_rn(b1, m[i]), __fmul_rn(1.0f - b1, gi));
  float vi = __fadd_rn(__fmul_rn(b2, v[i]), __fmul_rn(__fmul_rn(1.0f - b2, gi), gi));
  m[i] = mi;
  v[i] = vi;
  float mh = __fdiv_rn(mi, c1), vh = __fdiv_rn(vi, c2);
  theta[i] = __fsub_rn(theta[i], __fdiv_rn(__fmul_rn(lr, mh), __fadd_rn(__fsqrt_rn(vh), eps)));
}

}  // namespace

bool dgc_gemm_nt_persistent(const dgc_ctx *ctx, const float *a, int M, int N, int K) { return smallk_shape(ctx, a, M, N, K); }

// C[M][N] = A[M][K] * B[N][K]^T, no epilogue (used for the band -> tap map)
int32_t dgc_gemm_nt(dgc_ctx *ctx, const float *a, const float *b, int M, int N, int K, float *c) {
  int32_t rc = launch_sgemm<false, true, 0>(ctx, a, b, nullptr, M, N, K, c);
  if (rc != DGC_OK) return rc;
  ctx->launches++;
  return dgc_check_launch(ctx, "gemm_nt");
}

DGC_EXPORT int32_t dgc_linear_fwd(dgc_ctx *ctx, const float *a_dev, const float *w_dev, const float *bias_dev,
                                  int32_t M, int32_t K, int32_t N, int32_t act, float *c_dev, float *ct_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, a_dev && w_dev && c_dev, "null pointer");
  DGC_REQUIRE(ctx, M > 0 && K > 0 && N > 0, "size out of range");
  DGC_REQUIRE(ctx, act == 0 || act == 1, "act must be 0 (none) or 1 (tanh)");
  DGC_REQUIRE(ctx, act == 0 || bias_dev, "tanh layers need a bias");
  int32_t rc;
  bool ct_done = false;
  if (use_tensor_cores() && (double)M * N * K >= (double)(1 << 24) && (size_t)K * N <= (4u << 20) && (K & 3) == 0) {
    // The weight matrix is small next to the activations: transpose it once so that BOTH operands of the
    // tensor-core kernel are contiguous along k (vector loads straight into the K-major layout).
    if (!ctx->wt_buf || ctx->wt_floats < (uint64_t)K * N) {
      if (ctx->wt_buf) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(ctx->wt_buf);
        ctx->buffer_generation++;
        ctx->wt_buf = nullptr;
      }
      DGC_CUDA(ctx, cudaMalloc(&ctx->wt_buf, (size_t)K * N * sizeof(float)));
      ctx->wt_floats = (uint64_t)K * N;
    }
    transpose_kernel<<<dim3(dgc_div_up(N, 32), dgc_div_up(K, 32)), dim3(32, 8), 0, ctx->stream>>>(w_dev, K, N, ctx->wt_buf);
    DGC_LAUNCHED(ctx, "transpose_w");
    if (act == 1) rc = launch_sgemm<false, true, 2>(ctx, a_dev, ctx->wt_buf, bias_dev, M, N, K, c_dev, ct_dev, &ct_done);
    else if (bias_dev) rc = launch_sgemm<false, true, 1>(ctx, a_dev, ctx->wt_buf, bias_dev, M, N, K, c_dev, ct_dev, &ct_done);
    else rc = launch_sgemm<false, true, 0>(ctx, a_dev, ctx->wt_buf, nullptr, M, N, K, c_dev, ct_dev, &ct_done);
  } else if (K <= 4 && (N & 3) == 0 && ((((uintptr_t)w_dev) | ((uintptr_t)c_dev) | ((uintptr_t)bias_dev)) & 15) == 0) {
    // a handful of inputs: the streaming map
    const int64_t work = (int64_t)M * (N >> 2);
    const dim3 grid((unsigned)dgc_div_up(work, 256));
#define DGC_SMALLK_FWD(KKV)                                                                                           \
  do {                                                                                                               \
    if (act == 1) smallk_fwd_kernel<KKV, 2><<<grid, 256, 0, ctx->stream>>>(a_dev, w_dev, bias_dev, M, N, c_dev);      \
    else if (bias_dev) smallk_fwd_kernel<KKV, 1><<<grid, 256, 0, ctx->stream>>>(a_dev, w_dev, bias_dev, M, N, c_dev); \
    else smallk_fwd_kernel<KKV, 0><<<grid, 256, 0, ctx->stream>>>(a_dev, w_dev, nullptr, M, N, c_dev);                \
  } while (0)
    if (K == 1) DGC_SMALLK_FWD(1);
    else if (K == 2) DGC_SMALLK_FWD(2);
    else if (K == 3) DGC_SMALLK_FWD(3);
    else DGC_SMALLK_FWD(4);
#undef DGC_SMALLK_FWD
    rc = DGC_OK;
  } else
  if (act == 1) rc = launch_sgemm<false, false, 2>(ctx, a_dev, w_dev, bias_dev, M, N, K, c_dev);
  else if (bias_dev) rc = launch_sgemm<false, false, 1>(ctx, a_dev, w_dev, bias_dev, M, N, K, c_dev);
  else rc = launch_sgemm<false, false, 0>(ctx, a_dev, w_dev, nullptr, M, N, K, c_dev);
  if (rc != DGC_OK) return rc;
  DGC_LAUNCHED(ctx, "linear_fwd");
  if (ct_dev && !ct_done) {  // the matmul kernel that ran has no transposed store: one extra pass
    transpose_kernel<<<dim3(dgc_div_up(N, 32), dgc_div_up(M, 32)), dim3(32, 8), 0, ctx->stream>>>(c_dev, M, N, ct_dev);
    DGC_LAUNCHED(ctx, "transpose_c");
  }
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_linear_bwd(dgc_ctx *ctx, const float *a_dev, const float *w_dev, const float *c_dev,
                                  const float *dc_dev, int32_t M, int32_t K, int32_t N, int32_t act, float *dz_dev,
                                  float *da_dev, float *dw_dev, float *dbias_dev, const float *at_dev) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, a_dev && w_dev && dc_dev && dz_dev && dw_dev, "null pointer");
  DGC_REQUIRE(ctx, M > 0 && K > 0 && N > 0, "size out of range");
  DGC_REQUIRE(ctx, act == 0 || (act == 1 && c_dev), "tanh backward needs the layer output");
  const size_t n = (size_t)M * N;
  // With a transposed copy of the layer input at hand, the weight gradient reads both operands along the
  // reduction index m (the asynchronous K-major pipeline): dZ is then written in both orientations.
  const bool dw_kmajor = at_dev && use_tensor_cores() && (M & 3) == 0 && (double)M * N * K >= (double)(1 << 24) &&
                         (((uintptr_t)at_dev) & 15) == 0;
  if (dw_kmajor) {
    if (!ctx->dzt_buf || ctx->dzt_floats < n) {
      if (ctx->dzt_buf) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(ctx->dzt_buf);
        ctx->buffer_generation++;
        ctx->dzt_buf = nullptr;
      }
      DGC_CUDA(ctx, cudaMalloc(&ctx->dzt_buf, n * sizeof(float)));
      ctx->dzt_floats = n;
    }
    act_bwd_t_kernel<<<dim3(dgc_div_up(N, 32), dgc_div_up(M, 32)), dim3(32, 8), 0, ctx->stream>>>(dc_dev, c_dev, M, N, act,
                                                                                                dz_dev, ctx->dzt_buf);
  } else {
    const bool vec = (n & 3) == 0 && ((((uintptr_t)dc_dev) | ((uintptr_t)dz_dev) | (act == 1 ? (uintptr_t)c_dev : 0)) & 15) == 0;
    if (vec)
      act_bwd4_kernel<<<dgc_div_up((int64_t)(n / 4), 256), 256, 0, ctx->stream>>>(
          reinterpret_cast<const float4 *>(dc_dev), reinterpret_cast<const float4 *>(c_dev), n / 4, act,
          reinterpret_cast<float4 *>(dz_dev));
    else
      act_bwd_kernel<<<dgc_div_up((int64_t)n, 256), 256, 0, ctx->stream>>>(dc_dev, c_dev, n, act, dz_dev);
  }
  DGC_LAUNCHED(ctx, "act_bwd");
  const bool smallk = K <= 4;   // bias and weight gradient from one pass over dZ
  if (smallk) {
    const int chunks = dgc_div_up(M, 1024);
    float *part = dgc_ctx_scratch(ctx, (uint64_t)chunks * (K + 1) * N + 4);
    if (!part) return DGC_ERR_OOM;
    const dim3 grid(dgc_div_up(N, 32), chunks);
    if (K == 1) smallk_grad_kernel<1><<<grid, 256, 0, ctx->stream>>>(a_dev, dz_dev, M, N, part);
    else if (K == 2) smallk_grad_kernel<2><<<grid, 256, 0, ctx->stream>>>(a_dev, dz_dev, M, N, part);
    else if (K == 3) smallk_grad_kernel<3><<<grid, 256, 0, ctx->stream>>>(a_dev, dz_dev, M, N, part);
    else smallk_grad_kernel<4><<<grid, 256, 0, ctx->stream>>>(a_dev, dz_dev, M, N, part);
    DGC_LAUNCHED(ctx, "smallk_grad");
    smallk_grad_reduce_kernel<<<dgc_div_up((K + 1) * N, 128), 128, 0, ctx->stream>>>(part, chunks, K, N, dbias_dev, dw_dev);
    DGC_LAUNCHED(ctx, "smallk_grad_reduce");
  } else if (dbias_dev) {
    const int chunks = dgc_div_up(M, 1024);
    float *part = dgc_ctx_scratch(ctx, (uint64_t)chunks * N + 4);
    if (!part) return DGC_ERR_OOM;
    bias_grad_kernel<<<dim3(dgc_div_up(N, 32), chunks), 256, 0, ctx->stream>>>(dz_dev, M, N, part);
    DGC_LAUNCHED(ctx, "bias_grad");
    bias_grad_reduce_kernel<<<dgc_div_up(N, 128), 128, 0, ctx->stream>>>(part, chunks, N, dbias_dev);
    DGC_LAUNCHED(ctx, "bias_grad_reduce");
  }
  // dW[K][N] = A^T[K][M] * dZ[M][N]
  int32_t rc = smallk ? DGC_OK : dw_kmajor ? launch_sgemm<false, true, 0>(ctx, at_dev, ctx->dzt_buf, nullptr, K, N, M, dw_dev)
                         : launch_sgemm<true, false, 0>(ctx, a_dev, dz_dev, nullptr, K, N, M, dw_dev);
  if (rc != DGC_OK) return rc;
  if (!smallk) DGC_LAUNCHED(ctx, "linear_bwd_dw");
  if (da_dev) {
    // dA[M][K] = dZ[M][N] * W^T[N][K]
    rc = launch_sgemm<false, true, 0>(ctx, dz_dev, w_dev, nullptr, M, K, N, da_dev);
    if (rc != DGC_OK) return rc;
    DGC_LAUNCHED(ctx, "linear_bwd_da");
  }
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_adam_step(dgc_ctx *ctx, float *theta_dev, const float *grad_dev, float *m_dev, float *v_dev,
                                 uint64_t n, int32_t t, float lr, float beta1, float beta2, float eps) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, theta_dev && grad_dev && m_dev && v_dev, "null pointer");
  DGC_REQUIRE(ctx, t >= 1, "t is the 1-based step index");
  if (n == 0) return DGC_OK;
  // bias corrections as the reference computes them: 1 - pow(beta, Float(t)) in single precision
  float c1 = 1.0f - powf(beta1, (float)t), c2 = 1.0f - powf(beta2, (float)t);
  adam_kernel<<<dgc_div_up((int64_t)n, 256), 256, 0, ctx->stream>>>(theta_dev, grad_dev, m_dev, v_dev, n, lr, beta1,
                                                                    beta2, eps, c1, c2);
  DGC_LAUNCHED(ctx, "adam");
  return DGC_OK;
}

// The same step with the 1-based step index kept in device memory, so that a recorded step (graph.cu) advances it
// on every replay: a one-thread kernel increments *t_dev and evaluates the two bias corrections (in double, then
// rounded: the correctly rounded single-precision power), the update kernel reads them.
namespace {
__global__ void adam_tick_kernel(int32_t *t_dev, float beta1, float beta2, float *corr) {
  const int32_t t = *t_dev + 1;
  *t_dev = t;
  corr[0] = 1.0f - (float)pow((double)beta1, (double)t);
  corr[1] = 1.0f - (float)pow((double)beta2, (double)t);
}

__global__ void adam_counted_kernel(float *__restrict__ theta, const float *__restrict__ g, float *__restrict__ m,
                                    float *__restrict__ v, uint64_t n, float lr, float b1, float b2, float eps,
                                    const float *__restrict__ corr) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float c1 = corr[0], c2 = corr[1];
  float gi = g[i];
  float mi = __fadd_rn(__fmul_rn(b1, m[i]), __fmul_rn(1.0f - b1, gi));
  float vi = __fadd_rn(__fmul_rn(b2, v[i]), __fmul_rn(__fmul_rn(1.0f - b2, gi), gi));
  m[i] = mi;
  v[i] = vi;
  float mh = __fdiv_rn(mi, c1), vh = __fdiv_rn(vi, c2);
  theta[i] = __fsub_rn(theta[i], __fdiv_rn(__fmul_rn(lr, mh), __fadd_rn(__fsqrt_rn(vh), eps)));
}
}  // namespace

DGC_EXPORT int32_t dgc_adam_step_counted(dgc_ctx *ctx, float *theta_dev, const float *grad_dev, float *m_dev,
                                         float *v_dev, uint64_t n, int32_t *t_dev, float *corr_dev, float lr,
                                         float beta1, float beta2, float eps) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, theta_dev && grad_dev && m_dev && v_dev && t_dev && corr_dev, "null pointer");
  adam_tick_kernel<<<1, 1, 0, ctx->stream>>>(t_dev, beta1, beta2, corr_dev);
  DGC_LAUNCHED(ctx, "adam_tick");
  if (n == 0) return DGC_OK;
  adam_counted_kernel<<<dgc_div_up((int64_t)n, 256), 256, 0, ctx->stream>>>(theta_dev, grad_dev, m_dev, v_dev, n, lr,
                                                                            beta1, beta2, eps, corr_dev);
  DGC_LAUNCHED(ctx, "adam");
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_gemm_path_counts(dgc_ctx *ctx, int64_t *out4) {
  if (!ctx || !out4) return DGC_ERR_INVALID;
  for (int i = 0; i < 4; ++i) out4[i] = ctx->gemm_paths[i];
  return DGC_OK;
}

#ifdef DGC_KK_TIMING
DGC_EXPORT int32_t dgc_debug_kk_times(unsigned long long *out8) {
  cudaDeviceSynchronize();
  return cudaMemcpyFromSymbol(out8, dgtc::dgc_kk_times, 8 * sizeof(unsigned long long)) == cudaSuccess ? 0 : -1;
}
DGC_EXPORT int32_t dgc_debug_sk_times(unsigned long long *out128) {
  cudaDeviceSynchronize();
  return cudaMemcpyFromSymbol(out128, dgtc::dgc_sk_times, 128 * sizeof(unsigned long long)) == cudaSuccess ? 0 : -1;
}
#endif
