// fp32-accurate matmul on the 5th-generation tensor cores (tcgen05, accumulators in TMEM).
//
// C[M][N] = op(A)[M][K] * op(B)[K][N] in "3xTF32": every fp32 operand is split as x = hi + lo with hi the
// value the tensor core sees when it truncates x to TF32 and lo = x - hi (exact); the product is
// accumulated as hi*hi + hi*lo + lo*hi in fp32 in TMEM (missing term lo*lo ~ 2^-22 relative).
//
// One CTA (128 threads) owns a 128 x 128 output tile.  Per k-tile of 32 the four warps load the fp32
// operands from global memory, split them and store hi / lo parts to shared memory in the canonical
// K-major no-swizzle layout of the UMMA shared-memory descriptor (8-row x 16-byte core matrices; rows
// of a core matrix 16 bytes apart, 8-row groups SBO apart, 16-byte k-chunks LBO apart).  One elected
// thread issues 12 tcgen05.mma (4 k-steps of 8 x 3 products) and commits them to an mbarrier; two
// shared-memory stages let the loads of tile t+1 overlap the MMAs of tile t.  The epilogue reads the
// accumulators with tcgen05.ld (32 lanes x 32 columns per warp), applies bias / tanh and stores.
// Every wait on an mbarrier is bounded: on expiry the kernel raises the status word, and still frees
// its TMEM columns before returning.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dgtc {

constexpr int TBM = 128, TBN = 128, TBK = 32;
constexpr int CHUNKS = TBK / 4;                 // 16-byte k-chunks per row
constexpr int LBO_BYTES = TBM * 16 + 16;        // k-chunk stride (one 16-byte pad against bank conflicts)
constexpr int SBO_BYTES = 8 * 16;               // 8-row group stride
constexpr int OPER_BYTES = CHUNKS * LBO_BYTES;  // one operand part (hi or lo) of one stage
constexpr int STAGE_BYTES = 4 * OPER_BYTES;     // A_hi, A_lo, B_hi, B_lo
constexpr int SMEM_BYTES = 2 * STAGE_BYTES + 64;
constexpr uint32_t SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  // start address [0,14), leading byte offset [16,30), stride byte offset [32,46) (all >> 4),
  // descriptor version 1 at [46,48), layout type 0 (no swizzle) at [61,64)
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(LBO_BYTES >> 4) << 16) |
         ((uint64_t)(SBO_BYTES >> 4) << 32) | (1ull << 46);
}

// instruction descriptor: D = F32 (1 << 4), A = B = TF32 (2 << 7, 2 << 10), both K-major, N >> 3 at 17, M >> 4 at 24
constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TBN >> 3) << 17) | ((uint32_t)(TBM >> 4) << 24);

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
      "}\n" ::"r"(tmem_d), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate), "r"(0u)
      : "memory");
}

__device__ __forceinline__ void commit_to(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// true when the phase with the given parity has completed; bounded
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo) {
  hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
  lo = x - hi;
}

// element (row r, k index kk) of a K-major canonical operand part
__device__ __forceinline__ int oper_off(int r, int kk) { return (kk >> 2) * LBO_BYTES + r * 16 + (kk & 3) * 4; }

// Loads one 128 x 32 operand tile (rows r0.., k range k0..) and writes its hi / lo parts.
// ROWMAJOR_K: element (r, k) at src[r * ld + k] (k contiguous); else at src[k * ld + r] (r contiguous).
template <bool ROWMAJOR_K>
__device__ __forceinline__ void load_operand(const float *__restrict__ src, int ld, int rows, int r0, int k0, int k_end,
                                             char *hi_part, char *lo_part, int tid) {
  if (ROWMAJOR_K) {
    // 8 lanes cover the 8 k-chunks of a row (128 contiguous bytes), 16 rows per pass, 8 passes
    const int kc = tid & 7, rr = tid >> 3;
    const bool vec_ok = ((ld & 3) == 0) && ((((uintptr_t)src) & 15) == 0);
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      const int r = rr + 16 * p, gr = r0 + r, gk = k0 + 4 * kc;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (gr < rows) {
        const float *q = src + (size_t)gr * ld + gk;
        if (vec_ok && gk + 3 < k_end) v = *reinterpret_cast<const float4 *>(q);
        else {
          if (gk < k_end) v.x = q[0];
          if (gk + 1 < k_end) v.y = q[1];
          if (gk + 2 < k_end) v.z = q[2];
          if (gk + 3 < k_end) v.w = q[3];
        }
      }
      float4 h, l;
      split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
      const int off = kc * LBO_BYTES + r * 16;
      *reinterpret_cast<float4 *>(hi_part + off) = h;
      *reinterpret_cast<float4 *>(lo_part + off) = l;
    }
  } else {
    // r contiguous in memory: a warp reads 32 consecutive rows of one k (128 bytes); 4 warps take k = w, w+4, ...
    const int lane = tid & 31, w = tid >> 5;
#pragma unroll
    for (int kq = 0; kq < TBK / 4; ++kq) {
      const int kk = w + 4 * kq, gk = k0 + kk;
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const int r = lane + 32 * p, gr = r0 + r;
        float v = (gr < rows && gk < k_end) ? src[(size_t)gk * ld + gr] : 0.0f;
        float h, l;
        split_tf32(v, h, l);
        const int off = oper_off(r, kk);
        *reinterpret_cast<float *>(hi_part + off) = h;
        *reinterpret_cast<float *>(lo_part + off) = l;
      }
    }
  }
}

// A_KMAJOR: A stored [M][K]; else stored [K][M].  B_KMAJOR: B stored [N][K]; else stored [K][N].
// EPI 0: C = acc ; 1: + bias[n] ; 2: tanh(acc + bias[n]).  blockIdx.z selects a k-slice (split-K slab of C).
template <bool A_KMAJOR, bool B_KMAJOR, int EPI>
__global__ void __launch_bounds__(128, 1)
tc_gemm_kernel(const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ bias, int M, int N,
               int K, int k_per_split, float *__restrict__ C, int32_t *status) {
  extern __shared__ __align__(128) char smem[];
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + 2 * STAGE_BYTES);      // two mbarriers
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 2 * STAGE_BYTES + 32);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.y * TBM, n0 = blockIdx.x * TBN;
  const int k_begin = blockIdx.z * k_per_split, k_end = min(K, k_begin + k_per_split);
  C += (size_t)blockIdx.z * M * N;
  const int KT = (k_end - k_begin + TBK - 1) / TBK;

  if (tid == 0) {
    mbar_init(smem_u32(&bars[0]), 1);
    mbar_init(smem_u32(&bars[1]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)TBN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = *tmem_slot;
  bool ok = true;

  for (int kt = 0; kt < KT; ++kt) {
    const int s = kt & 1;
    if (kt >= 2) {
      ok = mbar_wait(smem_u32(&bars[s]), (uint32_t)(((kt >> 1) - 1) & 1));
      ok = __syncthreads_and(ok);   // same decision in every thread
      if (!ok) break;               // give up: no further MMAs are issued, TMEM is still released below
    }
    char *st = smem + s * STAGE_BYTES;
    const int k0 = k_begin + kt * TBK;
    load_operand<A_KMAJOR>(A, A_KMAJOR ? K : M, M, m0, k0, k_end, st, st + OPER_BYTES, tid);
    load_operand<B_KMAJOR>(B, B_KMAJOR ? K : N, N, n0, k0, k_end, st + 2 * OPER_BYTES, st + 3 * OPER_BYTES, tid);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> async proxy (tensor core)
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_hi = smem_u32(st), a_lo = a_hi + OPER_BYTES, b_hi = a_hi + 2 * OPER_BYTES, b_lo = a_hi + 3 * OPER_BYTES;
#pragma unroll
      for (int ks = 0; ks < TBK / 8; ++ks) {
        const uint32_t adv = ks * 2 * LBO_BYTES;  // 8 tf32 = two 16-byte k-chunks
        const uint64_t dah = make_desc(a_hi + adv), dal = make_desc(a_lo + adv);
        const uint64_t dbh = make_desc(b_hi + adv), dbl = make_desc(b_lo + adv);
        mma_tf32(tmem_d, dal, dbh, (kt | ks) ? 1u : 0u);   // small terms first
        mma_tf32(tmem_d, dah, dbl, 1u);
        mma_tf32(tmem_d, dah, dbh, 1u);
      }
      commit_to(smem_u32(&bars[s]));
    }
  }
  // the last commit covers every MMA issued before it
  if (KT > 0 && ok) ok = mbar_wait(smem_u32(&bars[(KT - 1) & 1]), (uint32_t)(((KT - 1) >> 1) & 1));
  ok = __syncthreads_and(ok);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  if (ok && KT > 0) {
    const int gm = m0 + warp * 32 + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < TBN; c0 += 32) {
      uint32_t r[32];
      const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
          "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
          "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
          : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
            "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
            "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
            "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
          : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (gm < M) {
        float *crow = C + (size_t)gm * N + n0 + c0;
        const bool vec_ok = ((N & 3) == 0) && (n0 + c0 + 31 < N) && ((((uintptr_t)C) & 15) == 0);
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float x = __uint_as_float(r[j + u]);
            int gn = n0 + c0 + j + u;
            if (EPI >= 1 && gn < N) x += bias[gn];
            if (EPI == 2) x = tanhf(x);
            v[u] = x;
          }
          if (vec_ok) *reinterpret_cast<float4 *>(crow + j) = make_float4(v[0], v[1], v[2], v[3]);
          else
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (n0 + c0 + j + u < N) crow[j + u] = v[u];
        }
      }
    }
  } else if (KT == 0) {
    // empty reduction range: the slab is zero
    const int gm = m0 + warp * 32 + lane;
    if (gm < M)
      for (int c = 0; c < TBN; ++c)
        if (n0 + c < N) C[(size_t)gm * N + n0 + c] = 0.0f;
  }
  if (!ok && tid == 0) atomicExch(status, 201);  // an MMA completion never arrived within the spin limit
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)TBN) : "memory");
  }
}

}  // namespace dgtc
