// fp32-accurate matmul on the 5th-generation tensor cores (tcgen05, accumulators in TMEM).
//
// C[M][N] = op(A)[M][K] * op(B)[K][N] in "3xTF32": every fp32 operand is split as x = hi + lo with hi the
// value the tensor core sees when it truncates x to TF32 and lo = x - hi (exact); the product is
// accumulated as hi*hi + hi*lo + lo*hi in fp32 in TMEM (missing term lo*lo ~ 2^-22 relative).
//
// One CTA (256 threads) owns a 128 x 128 output tile.  Per k-tile of 32 the eight warps load the fp32
// operands from global memory, split them and store hi / lo parts to shared memory in the canonical
// K-major no-swizzle layout of the UMMA shared-memory descriptor (8-row x 16-byte core matrices; rows of
// a core matrix 16 bytes apart, 8-row groups SBO apart, 16-byte k-chunks LBO apart); operands that are
// contiguous along m / n in memory are transposed on the way (vector loads, scalar stores).  One elected
// thread issues 12 tcgen05.mma (4 k-steps of 8 x 3 products) and commits them to an mbarrier; two
// shared-memory stages let the loads of tile t+1 overlap the MMAs of tile t.  The epilogue reads the
// accumulators with tcgen05.ld (32 lanes x 32 columns per warp), applies bias / tanh and stores.
// Every wait on an mbarrier is bounded: on expiry the kernel raises the status word, and still frees
// its TMEM columns before returning.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dgtc {

constexpr int TBM = 128, TBN = 128, TBK = 32, THREADS = 256;
constexpr int CHUNKS = TBK / 4;                 // 16-byte k-chunks per row
// K-major canonical layout (operand contiguous along k in memory): 16-byte unit (row r, k-chunk kc) at
// kc * LBO + r * 16; 8-row groups SBO = 128 bytes apart.
constexpr int LBO_BYTES = TBM * 16 + 16;        // k-chunk stride (one 16-byte pad against bank conflicts)
constexpr int SBO_BYTES = 8 * 16;               // 8-row group stride
// MN-major canonical layout (operand contiguous along m/n in memory): 16-byte unit = 4 consecutive m/n at one
// k, at (mn/4) * SBO_MN + (k % 8) * 16 + (k / 8) * LBO_MN (core matrix = 8 k-rows of 16 bytes, contiguous).
constexpr int SBO_MN_BYTES = 8 * 16;
constexpr int LBO_MN_BYTES = (TBM / 4) * SBO_MN_BYTES + 16;
// one operand part (hi or lo) of one stage: room for either layout
constexpr int OPER_BYTES = (CHUNKS * LBO_BYTES > (TBK / 8) * LBO_MN_BYTES) ? CHUNKS * LBO_BYTES : (TBK / 8) * LBO_MN_BYTES;
constexpr int STAGE_BYTES = 4 * OPER_BYTES;     // A_hi, A_lo, B_hi, B_lo
constexpr int SMEM_BYTES = 2 * STAGE_BYTES + 64;
constexpr uint32_t SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <bool KMAJOR>
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  // start address [0,14), leading byte offset [16,30), stride byte offset [32,46) (all >> 4),
  // descriptor version 1 at [46,48), layout type 0 (no swizzle) at [61,64)
  constexpr uint64_t lbo = KMAJOR ? LBO_BYTES : LBO_MN_BYTES, sbo = KMAJOR ? SBO_BYTES : SBO_MN_BYTES;
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((lbo >> 4) << 16) | ((sbo >> 4) << 32) | (1ull << 46);
}

// instruction descriptor: D = F32 (1 << 4), A = B = TF32 (2 << 7, 2 << 10), A / B major (0 = K, 1 = MN) at
// bits 15 / 16, N >> 3 at 17, M >> 4 at 24
template <bool A_KMAJOR, bool B_KMAJOR, int BN = TBN>
struct IDesc {
  static constexpr uint32_t value = (1u << 4) | (2u << 7) | (2u << 10) | (A_KMAJOR ? 0u : (1u << 15)) |
                                    (B_KMAJOR ? 0u : (1u << 16)) | ((uint32_t)(BN >> 3) << 17) |
                                    ((uint32_t)(TBM >> 4) << 24);
};

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t IDESC, uint32_t accumulate) {
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

// The same split with both parts ROUNDED to TF32 (round to nearest, ties away): |lo| <= 2^-11 |x| and what is
// lost, x - hi - lo, is at most 2^-22 |x| with either sign, where truncation loses up to 2^-20 |x| always
// towards zero (a bias that sums over a reduction instead of averaging out).
__device__ __forceinline__ void split_tf32_rn(float x, float &hi, float &lo) {
  // adding half a TF32 ulp to the bit pattern and clearing the 13 low bits rounds the magnitude to nearest, ties
  // away from zero (a carry into the exponent is the correct result); two integer instructions where the
  // conversion instruction runs at a quarter of their rate
  hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
  lo = __uint_as_float((__float_as_uint(x - hi) + 0x1000u) & 0xFFFFE000u);
}

// One 128 x 32 operand tile (rows r0.., k range k0..) moves in two steps so that the global loads of tile
// t+1 can be in flight while tile t is stored and multiplied: fetch() global memory -> 4 float4 registers
// per thread, stash() registers -> hi / lo parts in shared memory (256 threads).
// ROWMAJOR_K: element (r, k) at src[r * ld + k] (k contiguous): 8 lanes cover the 8 k-chunks of a row,
//   32 rows per pass, vector stores into the K-major layout.
// else: element at src[k * ld + r] (r contiguous): vector loads along m / n, transposed into the K-major
//   layout with scalar stores; a warp moves 8 k x 4 units (16 rows), a store instruction hits 8 k x 4 rows
//   with 2-way bank conflicts.  (An MN-major shared-memory descriptor with no swizzle was tried instead of
//   this transposition and produced zeros on this part, so both operands always use the K-major descriptor.)
template <bool ROWMAJOR_K>
__device__ __forceinline__ void fetch(const float *__restrict__ src, int ld, int rows, int r0, int k0, int k_end,
                                      int tid, float4 (&v)[4]) {
  const bool vec_ok = ((ld & 3) == 0) && ((((uintptr_t)src) & 15) == 0);
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    v[p] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ROWMAJOR_K) {
      const int kc = tid & 7, r = (tid >> 3) + 32 * p, gr = r0 + r, gk = k0 + 4 * kc;
      if (gr < rows) {
        const float *q = src + (size_t)gr * ld + gk;
        if (vec_ok && gk + 3 < k_end) v[p] = *reinterpret_cast<const float4 *>(q);
        else {
          if (gk < k_end) v[p].x = q[0];
          if (gk + 1 < k_end) v[p].y = q[1];
          if (gk + 2 < k_end) v[p].z = q[2];
          if (gk + 3 < k_end) v[p].w = q[3];
        }
      }
    } else {
      const int idx = p * THREADS + tid;
      const int kk = (idx & 7) + 8 * (idx >> 8), u = ((idx >> 3) & 3) + 4 * ((idx >> 5) & 7);
      const int gk = k0 + kk, gr = r0 + 4 * u;
      if (gk < k_end) {
        const float *q = src + (size_t)gk * ld + gr;
        if (vec_ok && gr + 3 < rows) v[p] = *reinterpret_cast<const float4 *>(q);
        else {
          if (gr < rows) v[p].x = q[0];
          if (gr + 1 < rows) v[p].y = q[1];
          if (gr + 2 < rows) v[p].z = q[2];
          if (gr + 3 < rows) v[p].w = q[3];
        }
      }
    }
  }
}

template <bool ROWMAJOR_K>
__device__ __forceinline__ void stash(const float4 (&v)[4], char *hi_part, char *lo_part, int tid) {
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    if (ROWMAJOR_K) {
      const int kc = tid & 7, r = (tid >> 3) + 32 * p;
      float4 h, l;
      split_tf32(v[p].x, h.x, l.x); split_tf32(v[p].y, h.y, l.y); split_tf32(v[p].z, h.z, l.z); split_tf32(v[p].w, h.w, l.w);
      const int off = kc * LBO_BYTES + r * 16;
      *reinterpret_cast<float4 *>(hi_part + off) = h;
      *reinterpret_cast<float4 *>(lo_part + off) = l;
    } else {
      const int idx = p * THREADS + tid;
      const int kk = (idx & 7) + 8 * (idx >> 8), u = ((idx >> 3) & 3) + 4 * ((idx >> 5) & 7);
      const float vv[4] = {v[p].x, v[p].y, v[p].z, v[p].w};
      const int base = (kk >> 2) * LBO_BYTES + (kk & 3) * 4 + (4 * u) * 16;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float h, l;
        split_tf32(vv[j], h, l);
        *reinterpret_cast<float *>(hi_part + base + j * 16) = h;
        *reinterpret_cast<float *>(lo_part + base + j * 16) = l;
      }
    }
  }
}

// tanh to ~1e-7 absolute in ~15 instructions (the library routine costs ~50 and dominated the epilogue):
// odd polynomial below 1/4 (next term 62/2835 x^9 < 1e-7 relative there), 1 - 2 / (e^{2|x|} + 1) above.
__device__ __forceinline__ float tanh_fast(float x) {
  const float ax = fabsf(x), x2 = x * x;
  const float p = x * fmaf(x2, fmaf(x2, fmaf(x2, -17.0f / 315.0f, 2.0f / 15.0f), -1.0f / 3.0f), 1.0f);
  const float e = __expf(2.0f * fminf(ax, 15.0f));
  const float t = copysignf(1.0f - __fdividef(2.0f, e + 1.0f), x);
  return ax < 0.25f ? p : t;
}

constexpr int EPI_STAGE_FLOATS = 32 * 33;   // per warp: a 32 x 32 block, rows padded to 33 floats

// Accumulators -> global memory.  Warp w may touch tensor-memory lanes 32 * (w % 4) ..; warps 0-3 take columns
// 0..63, warps 4-7 the rest; after tcgen05.ld a lane holds 32 columns of ONE output row.  Storing from there
// would make every store instruction touch 32 different rows, so each warp turns its 32 x 32 block through a
// private shared-memory tile (`stage`, EPI_STAGE_FLOATS floats per warp, the pipeline's buffers are idle by
// now) and writes full 128-byte row segments.  EPI 0: C = acc ; 1: + bias[n] ; 2: tanh(acc + bias[n]).
// Ct (optional): a second, transposed copy Ct[n][m] of the result, written straight from the registers
// (lanes = consecutive m: already 128-byte stores).
template <int EPI, int BN = TBN>
__device__ __forceinline__ void epilogue(uint32_t tmem_d, const float *__restrict__ bias, int M, int N, int m0, int n0,
                                         float *__restrict__ C, int warp, int lane, float *__restrict__ Ct,
                                         float *__restrict__ stage_all) {
  const int lane_base = (warp & 3) * 32, col_base = (warp >> 2) * (BN / 2);
  const int gm = m0 + lane_base + lane;
  float *stage = stage_all + warp * EPI_STAGE_FLOATS;
  const bool aligned = ((N & 3) == 0) && ((((uintptr_t)C) & 15) == 0);
#pragma unroll 1
  for (int c0 = col_base; c0 < col_base + BN / 2; c0 += 32) {
    if (n0 + c0 >= N) break;   // the rest of this tile lies beyond the last column (warp-uniform)
    uint32_t r[32];
    const uint32_t taddr = tmem_d + ((uint32_t)lane_base << 16) + (uint32_t)c0;
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
    const int gn0 = n0 + c0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float x = __uint_as_float(r[j]);
      if (EPI >= 1 && gn0 + j < N) x += __ldg(&bias[gn0 + j]);
      if (EPI == 2) x = tanh_fast(x);
      if (Ct && gm < M && gn0 + j < N) Ct[(size_t)(gn0 + j) * M + gm] = x;
      stage[lane * 33 + j] = x;   // bank (lane + j) % 32: conflict-free
    }
    __syncwarp();
    const bool vec_ok = aligned && gn0 + 31 < N;
    if (vec_ok) {
      // 4 rows per instruction: lane -> (row it * 4 + lane / 8, columns 4 * (lane % 8) ..)
      const int rsub = lane >> 3, c4 = (lane & 7) * 4;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int rr = it * 4 + rsub, grow = m0 + lane_base + rr;
        const float *sp = stage + rr * 33 + c4;
        const float v0 = sp[0], v1 = sp[1], v2 = sp[2], v3 = sp[3];
        if (grow < M) *reinterpret_cast<float4 *>(C + (size_t)grow * N + gn0 + c4) = make_float4(v0, v1, v2, v3);
      }
    } else {
      // rows that are not 16-byte aligned (N not a multiple of 4) or the ragged last columns: one row per
      // instruction, lanes = consecutive columns, so every store still covers one contiguous run of a row
      const bool col_ok = gn0 + lane < N;
#pragma unroll 8
      for (int rr = 0; rr < 32; ++rr) {
        const int grow = m0 + lane_base + rr;
        const float v = stage[rr * 33 + lane];
        if (col_ok && grow < M) C[(size_t)grow * N + gn0 + lane] = v;
      }
    }
    __syncwarp();
  }
}

// A_KMAJOR: A stored [M][K]; else stored [K][M].  B_KMAJOR: B stored [N][K]; else stored [K][N].
// EPI 0: C = acc ; 1: + bias[n] ; 2: tanh(acc + bias[n]).  blockIdx.z selects a k-slice (split-K slab of C).
template <bool A_KMAJOR, bool B_KMAJOR, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
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

  float4 va[4], vb[4], na[4], nb[4];
  if (KT > 0) {
    fetch<A_KMAJOR>(A, A_KMAJOR ? K : M, M, m0, k_begin, k_end, tid, va);
    fetch<B_KMAJOR>(B, B_KMAJOR ? K : N, N, n0, k_begin, k_end, tid, vb);
  }
  for (int kt = 0; kt < KT; ++kt) {
    const int s = kt & 1;
    if (kt + 1 < KT) {  // next tile's global loads fly while this tile is stored and multiplied
      fetch<A_KMAJOR>(A, A_KMAJOR ? K : M, M, m0, k_begin + (kt + 1) * TBK, k_end, tid, na);
      fetch<B_KMAJOR>(B, B_KMAJOR ? K : N, N, n0, k_begin + (kt + 1) * TBK, k_end, tid, nb);
    }
    if (kt >= 2) {
      ok = mbar_wait(smem_u32(&bars[s]), (uint32_t)(((kt >> 1) - 1) & 1));
      ok = __syncthreads_and(ok);   // same decision in every thread
      if (!ok) break;               // give up: no further MMAs are issued, TMEM is still released below
    }
    char *st = smem + s * STAGE_BYTES;
    stash<A_KMAJOR>(va, st, st + OPER_BYTES, tid);
    stash<B_KMAJOR>(vb, st + 2 * OPER_BYTES, st + 3 * OPER_BYTES, tid);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> async proxy (tensor core)
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_hi = smem_u32(st), a_lo = a_hi + OPER_BYTES, b_hi = a_hi + 2 * OPER_BYTES, b_lo = a_hi + 3 * OPER_BYTES;
      constexpr uint32_t ID = IDesc<true, true>::value;
#pragma unroll
      for (int ks = 0; ks < TBK / 8; ++ks) {
        // 8 tf32 along k = two 16-byte k-chunks
        const uint32_t adv = ks * 2 * LBO_BYTES;
        const uint64_t dah = make_desc<true>(a_hi + adv), dal = make_desc<true>(a_lo + adv);
        const uint64_t dbh = make_desc<true>(b_hi + adv), dbl = make_desc<true>(b_lo + adv);
        mma_tf32(tmem_d, dal, dbh, ID, (kt | ks) ? 1u : 0u);   // small terms first
        mma_tf32(tmem_d, dah, dbl, ID, 1u);
        mma_tf32(tmem_d, dah, dbh, ID, 1u);
      }
      commit_to(smem_u32(&bars[s]));
    }
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      va[p] = na[p];
      vb[p] = nb[p];
    }
  }
  // the last commit covers every MMA issued before it
  if (KT > 0 && ok) ok = mbar_wait(smem_u32(&bars[(KT - 1) & 1]), (uint32_t)(((KT - 1) >> 1) & 1));
  ok = __syncthreads_and(ok);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  if (ok && KT > 0) {
    epilogue<EPI>(tmem_d, bias, M, N, m0, n0, C, warp, lane, nullptr, reinterpret_cast<float *>(smem));
  } else if (KT == 0) {
    // empty reduction range: the slab is zero
    const int gm = m0 + (warp & 3) * 32 + lane;
    if (gm < M && warp < 4)
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


// ---------------------------------------------------------------------------------------------------------
// Both operands contiguous along k in memory (A [M][K], B [N][K]), K a multiple of 4, 16-byte aligned rows:
// the asynchronous pipeline.  cp.async copies 16-byte chunks straight into the canonical K-major layout,
// RAW raw stages deep, PF tiles ahead of the tensor core; the raw fp32 tile IS the "hi" operand (the tensor
// core reads the top 19 bits of every 32-bit word and ignores the 13 low mantissa bits, i.e. it truncates
// to TF32 itself), so the threads only compute lo = x - trunc(x), shared memory to shared memory, into one
// of two lo buffers.  Tile t's MMAs commit to an mbarrier of their own raw stage; the only wait of
// iteration t is on tile t-2 (it frees both the raw stage about to be refilled and the lo buffer about to
// be rewritten), two iterations after its MMAs were issued.
// ---------------------------------------------------------------------------------------------------------
// SW: the 128-byte-swizzle K-major layout (BK = 32: one row of a tile is exactly one 128-byte swizzle row;
// 8-row groups of 1024 bytes, 16-byte chunk c of row r stored at chunk c ^ (r % 8)) instead of the
// no-swizzle layout of 8 x 16-byte core matrices.
// With BK = 16 a row is 64 bytes and the 64-byte swizzle applies (8-row groups of 512 bytes, chunk c of row r at
// c ^ ((r / 2) % 4)); that variant needs 97 KB per CTA, so two CTAs share an SM and one's epilogue runs under
// the other's main loop.
// BN = 256 (swizzled layouts only): a 128 x 256 output tile per CTA.  Per flop the three MMAs of a k step then
// fetch 25 % fewer operand bytes (A is shared by twice as many columns) and the copy / split traffic drops by
// the same factor, which is what the kernel is bound by; 145 KB of shared memory, one CTA per SM.
template <int BK, bool SW = false, int BN = TBN>
struct KK {
  static_assert(BN == TBN || SW, "the wide tile uses the swizzled layouts");
  static constexpr int CHUNKS_K = BK / 4;
  static constexpr int ROW_BYTES = BK * 4;                                  // 128 or 64
  static constexpr int OPER = SW ? TBM * ROW_BYTES : CHUNKS_K * LBO_BYTES;  // operand A of one tile
  static constexpr int OPER_B = SW ? BN * ROW_BYTES : CHUNKS_K * LBO_BYTES; // operand B of one tile
  static constexpr int RAW = 4, PF = 2;
  static constexpr int RAW_STAGE = OPER + OPER_B;         // A, B
  static constexpr int SMEM = (RAW + 2) * RAW_STAGE + 128 + (SW ? 1024 : 0);   // + room to align to 1024
  // byte offset of 16-byte chunk kc of row r inside one operand
  __device__ static __forceinline__ int unit_offset(int r, int kc) {
    if (!SW) return kc * LBO_BYTES + r * 16;
    return BK == 32 ? (r >> 3) * 1024 + (r & 7) * 128 + ((kc ^ (r & 7)) << 4)
                    : (r >> 3) * 512 + (r & 7) * 64 + ((kc ^ ((r >> 1) & 3)) << 4);
  }
  static constexpr int UNITS = (TBM + BN) * CHUNKS_K;     // 16-byte units per tile (A and B)
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// one float; src_bytes 0 = zero fill.  For operands whose rows are not 16-byte aligned (K not a multiple of 4).
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// K-major, 128-byte swizzle: LBO unused (1), SBO = 1024 bytes between 8-row groups, layout type 2 at [61,64)
// (64-byte swizzle: SBO = 512 bytes, layout type 4)
template <int ROW_BYTES = 128>
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr) {
  constexpr uint64_t sbo = ROW_BYTES * 8, type = ROW_BYTES == 128 ? 2 : 4;
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((sbo >> 4) << 32) | (1ull << 46) | (type << 61);
}

#ifdef DGC_KK_TIMING
// development aid: per-phase timestamps (ns) of CTA (0,0,0), read back with cudaMemcpyFromSymbol
__device__ unsigned long long dgc_kk_times[8];
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define KK_STAMP(i) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x & 31) == 0 && (threadIdx.x == 0 || (i) == 3 || (i) == 4)) dgc_kk_times[i] = gtime(); } while (0)
#else
#define KK_STAMP(i) do {} while (0)
#endif

constexpr int KK_THREADS = THREADS + 32;   // 8 worker warps + 1 warp whose lane 0 issues the MMAs

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// A4: the operands' rows are only 4-byte aligned (K % 4 != 0): every 16-byte unit is fetched as four 4-byte copies.
template <int EPI, int BK, bool SW, int BN = TBN, bool A4 = false>
__global__ void __launch_bounds__(KK_THREADS, (BK == 16 && BN == TBN) ? 2 : 1)
tc_gemm_kk_kernel(const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ bias, int M, int N,
                  int K, int k_per_split, float *__restrict__ C, float *__restrict__ Ct, int32_t *status) {
  using G = KK<BK, SW, BN>;
  KK_STAMP(0);
  extern __shared__ __align__(128) char smem_base[];
  // the swizzle pattern is a function of the address: tiles start on 1024-byte boundaries
  char *smem = SW ? smem_base + ((1024u - (smem_u32(smem_base) & 1023u)) & 1023u) : smem_base;
  char *raw = smem, *lob = smem + G::RAW * G::RAW_STAGE;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (G::RAW + 2) * G::RAW_STAGE);  // RAW "tile consumed" mbarriers
  uint64_t *ready = bars + G::RAW;                                                    // 2 "lo buffer written" mbarriers
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (G::RAW + 2) * G::RAW_STAGE + 64);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.y * TBM, n0 = blockIdx.x * BN;
  const int k_begin = blockIdx.z * k_per_split, k_end = min(K, k_begin + k_per_split);
  C += (size_t)blockIdx.z * M * N;
  const int KT = (k_end - k_begin + BK - 1) / BK;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < G::RAW; ++i) mbar_init(smem_u32(&bars[i]), 1);
    mbar_init(smem_u32(&ready[0]), THREADS / 32);   // one arrival per worker warp
    mbar_init(smem_u32(&ready[1]), THREADS / 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)BN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = *tmem_slot;
  bool ok = true;

  volatile int *failed = reinterpret_cast<volatile int *>(tmem_slot + 1);
  if (tid == 0) *failed = 0;
  __syncthreads();
  KK_STAMP(1);

  if (warp < THREADS / 32) {
    // ---- worker warps: copy, split, publish -----------------------------------------------------------------
    // This thread's share of every tile: units u = tid + 256 * i -> (operand, row, k-chunk), chunk fastest, so 8
    // lanes fetch one 128-byte row.  Global pointers and shared offsets are fixed per thread, and the thread
    // splits exactly the units it copied itself, so the only synchronisation of the loop is through mbarriers:
    // "tile kt-2 consumed" before its raw stage and lo buffer are reused, "lo buffer written" towards the MMA warp.
    constexpr int UPT = G::UNITS / THREADS;
    const float *src0[UPT];
    int soff[UPT], kc4[UPT];
    bool rowok[UPT];
#pragma unroll
    for (int i = 0; i < UPT; ++i) {
      const int u = tid + THREADS * i;
      const int op = u >= TBM * G::CHUNKS_K, rem = u - op * (TBM * G::CHUNKS_K);   // A units first, then B
      const int r = rem / G::CHUNKS_K, kc = rem % G::CHUNKS_K;
      const int rows = op ? N : M, gr = (op ? n0 : m0) + r;
      rowok[i] = gr < rows;
      kc4[i] = 4 * kc;
      src0[i] = (op ? B : A) + (rowok[i] ? (size_t)gr * K : 0) + k_begin + 4 * kc;
      soff[i] = op * G::OPER + G::unit_offset(r, kc);
    }
    // A4 (rows only 4-byte aligned): the tile is copied float by float, element e = tid + 256 i -> (row e / BK,
    // k = e % BK), so the lanes of a warp copy consecutive floats of two rows (a unit-wise assignment would
    // make every instruction touch eight rows).  256 % BK == 0: k is the same for all of a thread's elements, its
    // rows are 16 apart, and each element's place in shared memory moves by a constant from one to the next.
    static_assert(!A4 || (BK == 16 && BN == TBN), "the 4-byte copy path is written for 16-wide k tiles and 128 columns");
    constexpr int EPT4 = (TBM + BN) * BK / THREADS;          // 16 elements per thread: 8 of A, 8 of B
    const int k4 = tid % BK, r4 = tid / BK;                  // A4: this thread's k and first row
    const int soff4 = G::unit_offset(r4, k4 >> 2) + (k4 & 3) * 4;
    const int dsoff4 = G::unit_offset(r4 + THREADS / BK, k4 >> 2) - G::unit_offset(r4, k4 >> 2);
    auto issue_tile = [&](int kt) {
      if (kt < KT) {
        const int k0 = kt * BK;   // relative to k_begin
        const uint32_t st = smem_u32(raw + (kt % G::RAW) * G::RAW_STAGE);
        if (A4) {
          const bool kin = k_begin + k0 + k4 < k_end;
#pragma unroll
          for (int i = 0; i < EPT4; ++i) {
            const int op = i >= EPT4 / 2, r = r4 + (THREADS / BK) * (i - op * (EPT4 / 2));
            const int gr = (op ? n0 : m0) + r;
            const bool in = kin && gr < (op ? N : M);
            cp_async4(st + op * G::OPER + soff4 + (i - op * (EPT4 / 2)) * dsoff4,
                      in ? (op ? B : A) + (size_t)gr * K + k_begin + k0 + k4 : A, in ? 4 : 0);
          }
        } else {
#pragma unroll
          for (int i = 0; i < UPT; ++i) {
            int bytes = (k_end - k_begin - k0 - kc4[i]) * 4;
            bytes = rowok[i] ? (bytes > 16 ? 16 : (bytes < 0 ? 0 : bytes)) : 0;
            cp_async16(st + soff[i], bytes > 0 ? src0[i] + k0 : A, bytes);   // 0 bytes: zero fill, any valid address
          }
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");   // one group per call keeps the counting uniform
    };
#pragma unroll
    for (int p = 0; p < G::PF; ++p) issue_tile(p);
    for (int kt = 0; kt < KT; ++kt) {
      if (kt >= 2 && !*failed) {   // bounded; a thread that gives up raises the shared flag and everybody stops waiting
        if (!mbar_wait(smem_u32(&bars[(kt - 2) % G::RAW]), (uint32_t)(((kt - 2) / G::RAW) & 1))) *failed = 1;
      }
      issue_tile(kt + G::PF);
      asm volatile("cp.async.wait_group %0;" ::"n"(G::PF) : "memory");   // this thread's chunks of tile kt landed
      if (kt == 0) KK_STAMP(2);
      char *st = raw + (kt % G::RAW) * G::RAW_STAGE, *lo = lob + (kt & 1) * G::RAW_STAGE;
      if (A4) {
        float v[EPT4];
#pragma unroll
        for (int i = 0; i < EPT4; ++i)
          v[i] = *reinterpret_cast<const float *>(st + (i >= EPT4 / 2) * G::OPER + soff4 + (i % (EPT4 / 2)) * dsoff4);
#pragma unroll
        for (int i = 0; i < EPT4; ++i) {
          float h, l;
          split_tf32(v[i], h, l);
          *reinterpret_cast<float *>(lo + (i >= EPT4 / 2) * G::OPER + soff4 + (i % (EPT4 / 2)) * dsoff4) = l;
        }
      } else {
#pragma unroll
        for (int i = 0; i < UPT; ++i) {
          const float4 v = *reinterpret_cast<const float4 *>(st + soff[i]);
          float4 h, l;
          split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
          *reinterpret_cast<float4 *>(lo + soff[i]) = l;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // this thread's writes -> tensor-core proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ready[kt & 1]));
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (lane == 0) {
    // ---- MMA issue: one thread, nothing else to do ----------------------------------------------------------
    constexpr uint32_t ID = IDesc<true, true, BN>::value;
    for (int kt = 0; kt < KT; ++kt) {
      if (*failed || !mbar_wait(smem_u32(&ready[kt & 1]), (uint32_t)((kt >> 1) & 1))) {
        *failed = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (kt == 0) KK_STAMP(3);
      const uint32_t a_hi = smem_u32(raw + (kt % G::RAW) * G::RAW_STAGE), b_hi = a_hi + G::OPER;
      const uint32_t a_lo = smem_u32(lob + (kt & 1) * G::RAW_STAGE), b_lo = a_lo + G::OPER;
#pragma unroll
      for (int ks = 0; ks < BK / 8; ++ks) {
        // 8 tf32 along k: two 16-byte chunks (no swizzle), or 32 bytes further inside the swizzled row
        const uint32_t adv = SW ? ks * 32 : ks * 2 * LBO_BYTES;
        const uint64_t dah = SW ? make_desc_sw128<G::ROW_BYTES>(a_hi + adv) : make_desc<true>(a_hi + adv);
        const uint64_t dal = SW ? make_desc_sw128<G::ROW_BYTES>(a_lo + adv) : make_desc<true>(a_lo + adv);
        const uint64_t dbh = SW ? make_desc_sw128<G::ROW_BYTES>(b_hi + adv) : make_desc<true>(b_hi + adv);
        const uint64_t dbl = SW ? make_desc_sw128<G::ROW_BYTES>(b_lo + adv) : make_desc<true>(b_lo + adv);
        mma_tf32(tmem_d, dal, dbh, ID, (kt | ks) ? 1u : 0u);
        mma_tf32(tmem_d, dah, dbl, ID, 1u);
        mma_tf32(tmem_d, dah, dbh, ID, 1u);
      }
      commit_to(smem_u32(&bars[kt % G::RAW]));
    }
    // the last commit covers every MMA issued before it
    if (KT > 0 && !*failed && !mbar_wait(smem_u32(&bars[(KT - 1) % G::RAW]), (uint32_t)(((KT - 1) / G::RAW) & 1)))
      *failed = 1;
    KK_STAMP(4);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  ok = !*failed;
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  KK_STAMP(5);

  if (ok && KT > 0) {
    if (warp < THREADS / 32) epilogue<EPI, BN>(tmem_d, bias, M, N, m0, n0, C, warp, lane, Ct, reinterpret_cast<float *>(smem));
    KK_STAMP(6);
  } else if (KT == 0) {
    const int gm = m0 + (warp & 3) * 32 + lane;
    if (gm < M && warp < 4)
      for (int c = 0; c < BN; ++c)
        if (n0 + c < N) C[(size_t)gm * N + n0 + c] = 0.0f;
  }
  if (!ok && tid == 0) atomicExch(status, 201);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)BN) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------
// Short reductions (K <= 72; the band -> tap map has K = 65, N = 257): A [M][K], B [N][K], both contiguous
// along k.  With so few k-tiles a CTA per output tile spends its life in prologue, load latency and epilogue,
// so this kernel is persistent: a CTA owns ONE 128-column block of the output, keeps that block of B (hi and
// lo parts) in shared memory for its whole life and walks down the row tiles of A.
//   copy     a 128-row tile of A is one contiguous, 16-byte aligned run of 128 K floats whatever K's alignment:
//            the thread that issues the MMAs fetches it with ONE bulk copy (cp.async.bulk, completion on an
//            mbarrier) into a linear staging buffer, as soon as the previous tile has been split out of it
//   split    sixteen worker warps read the linear tile and write its hi and lo parts (both rounded to TF32) into
//            the K-major no-swizzle layout of make_desc<true>(): 16-byte unit (row r, chunk kc) at
//            kc * LBO_BYTES + r * 16; k is padded to a multiple of 8 with zeros that are written once
//   multiply one thread issues the 3 x ceil(K / 8) MMAs of the tile into one of TWO 128-column accumulators
//   store    while the tensor core works on tile i, the worker warps move tile i-1 from the other accumulator to
//            global memory (32 x 16 blocks turned through shared memory into 64-byte row segments)
// N % 128 <= SK::EXTRA_MAX leftover columns (the 257th tap) are plain fp32 dot products of the CTAs of the
// last column block, from the linear tile, instead of a third block of 127 empty columns.
// Every wait is bounded; on expiry the kernel raises status 202, stops waiting everywhere and frees its TMEM.
// ---------------------------------------------------------------------------------------------------------
#ifdef DGC_KK_TIMING
__device__ unsigned long long dgc_sk_times[128];
#define SK_STAMP(i) do { if (tid == 0 && blockIdx.x == 0 && (i) < 128) dgc_sk_times[(i)] = gtime(); } while (0)
#else
#define SK_STAMP(i) do {} while (0)
#endif
struct SK {
  static constexpr int KP_MAX = 72;                          // largest K (nine k-steps of 8)
  static constexpr int WORKERS = 512, THREADS_ALL = WORKERS + 32;
  static constexpr int OPER = (KP_MAX / 4) * LBO_BYTES;      // one operand part: 18 chunks
  static constexpr int OFF_BHI = 0, OFF_BLO = OPER, OFF_AHI = 2 * OPER, OFF_ALO = 3 * OPER, OFF_LIN = 4 * OPER;
  static constexpr int LIN_BYTES = TBM * KP_MAX * 4;
  static constexpr int EPI_ROW = 20;                         // floats per staged row of 16 (16-byte stores, no conflicts)
  static constexpr int OFF_STAGE = OFF_LIN + LIN_BYTES;
  static constexpr int OFF_BARS = OFF_STAGE + (WORKERS / 32) * 32 * EPI_ROW * 4;
  static constexpr int SMEM = OFF_BARS + 64;
  static constexpr int EPT = TBM * KP_MAX / WORKERS;         // elements of a tile per worker thread
  static constexpr int EXTRA_MAX = 8;
};
static_assert(SK::SMEM <= 227 * 1024, "the persistent small-K kernel must fit one CTA's shared memory");
static_assert(SK::OFF_LIN % 128 == 0 && SK::OFF_STAGE % 16 == 0 && SK::OFF_BARS % 8 == 0, "alignment of the buffers");

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// linear global -> shared copy by the copy engine; both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__global__ void __launch_bounds__(SK::THREADS_ALL, 1)
tc_gemm_smallk_kernel(const float *__restrict__ A, const float *__restrict__ B, int M, int N, int K, int nblk,
                      int n_extra, int ctas_per_blk, float *__restrict__ C, int32_t *status) {
  extern __shared__ __align__(128) char smem[];
  char *b_hi = smem + SK::OFF_BHI, *b_lo = smem + SK::OFF_BLO, *a_hi = smem + SK::OFF_AHI, *a_lo = smem + SK::OFF_ALO;
  float *lin = reinterpret_cast<float *>(smem + SK::OFF_LIN);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + SK::OFF_BARS);
  const uint32_t bar_ready = smem_u32(bars), bar_done = smem_u32(bars + 1), bar_load = smem_u32(bars + 2);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + SK::OFF_BARS + 32);
  volatile int *failed = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cb = blockIdx.x % nblk, slot = blockIdx.x / nblk;
  const int n0 = cb * TBN;
  const int row_tiles = (M + TBM - 1) / TBM;
  const int nt = (row_tiles - slot + ctas_per_blk - 1) / ctas_per_blk;   // row tiles slot, slot + ctas_per_blk, ...
  const bool has_extra = n_extra > 0 && cb == nblk - 1;
  const int ksteps = (K + 7) / 8;
  const int tile_elems = TBM * K;

  // zeros once: the k padding of all four operand parts and the rows past the end of B are never written again
  for (int u = tid; u < SK::OFF_LIN / 16; u += SK::THREADS_ALL)
    reinterpret_cast<float4 *>(smem)[u] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (tid == 0) {
    mbar_init(bar_ready, SK::WORKERS / 32);   // one arrival per worker warp
    mbar_init(bar_done, 1);
    mbar_init(bar_load, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    *failed = 0;
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)(2 * TBN))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = *tmem_slot;
  SK_STAMP(0);

  if (warp < SK::WORKERS / 32) {
    // ---- worker warps ---------------------------------------------------------------------------------------
    // element e = tid + 512 j of a tile is (row e / K, k = e % K); its byte offset inside an operand part is the
    // same for A and B and fixed for the life of the thread
    unsigned short off[SK::EPT];
    {
      int r = tid / K, k = tid - r * K;
      const int dr = SK::WORKERS / K, dk = SK::WORKERS - dr * K;
#pragma unroll
      for (int j = 0; j < SK::EPT; ++j) {
        off[j] = (unsigned short)((k >> 2) * LBO_BYTES + r * 16 + (k & 3) * 4);   // < 65536 (rows past 127: unused)
        r += dr; k += dk;
        if (k >= K) { k -= K; ++r; }
      }
    }
    // this CTA's block of B, split once
    {
      const size_t b0 = (size_t)n0 * K, bend = (size_t)N * K;
#pragma unroll
      for (int j = 0; j < SK::EPT; ++j) {
        const int e = tid + SK::WORKERS * j;
        if (e < tile_elems && b0 + e < bend) {
          float h, l;
          split_tf32_rn(__ldg(B + b0 + e), h, l);
          *reinterpret_cast<float *>(b_hi + off[j]) = h;
          *reinterpret_cast<float *>(b_lo + off[j]) = l;
        }
      }
    }
    // accumulator i & 1 -> C, after the MMAs of tile i completed.  Warp w may read tensor-memory lanes
    // 32 (w % 4) ..; it takes columns 32 (w / 4) .. of them, sixteen at a time: after tcgen05.ld a lane holds 16
    // columns of ONE row, the block is turned through the warp's private staging rows, and every store
    // instruction writes two 64-byte row segments.
    float *stage = reinterpret_cast<float *>(smem + SK::OFF_STAGE) + warp * 32 * SK::EPI_ROW;
    auto store_tile = [&](int i) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int lane_base = (warp & 3) * 32, m0 = (slot + i * ctas_per_blk) * TBM;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c0 = (warp >> 2) * 32 + 16 * h, gn0 = n0 + c0;
        if (gn0 >= N) break;   // warp-uniform: the rest of this block lies beyond the last column
        uint32_t r[16];
        const uint32_t taddr = tmem_d + (uint32_t)((i & 1) * TBN) + ((uint32_t)lane_base << 16) + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (h == 0) SK_STAMP(8 + 8 * (i + 1));
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4 *>(stage + lane * SK::EPI_ROW + 4 * q) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        __syncwarp();
        // an instruction stores rows r and r + 4: 4 x 20 floats apart, i.e. 16 banks apart, so the two 16-float
        // segments it reads from the staging rows cover all 32 banks once
        const int rsub = lane >> 4, col = lane & 15;
        const bool col_ok = gn0 + col < N;
        float v[16];
#pragma unroll
        for (int it = 0; it < 16; ++it) v[it] = stage[((it & 3) + 8 * (it >> 2) + 4 * rsub) * SK::EPI_ROW + col];
        if (h == 0) SK_STAMP(9 + 8 * (i + 1));
#pragma unroll
        for (int it = 0; it < 16; ++it) {
          const int grow = m0 + lane_base + (it & 3) + 8 * (it >> 2) + 4 * rsub;
          if (col_ok && grow < M) C[(size_t)grow * N + gn0 + col] = v[it];
        }
        if (h == 0) SK_STAMP(10 + 8 * (i + 1));
        __syncwarp();
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      SK_STAMP(11 + 8 * (i + 1));
    };
    SK_STAMP(1);
    for (int i = 0; i < nt; ++i) {
      // tile i has landed in the linear buffer; tile i-1 is multiplied: its accumulator is complete and the
      // operand parts of A may be overwritten
      if (!*failed && !mbar_wait(bar_load, (uint32_t)(i & 1))) *failed = 1;
      SK_STAMP(4 + 8 * i);
      if (i >= 1 && !*failed && !mbar_wait(bar_done, (uint32_t)((i - 1) & 1))) *failed = 1;
      SK_STAMP(5 + 8 * i);
      if (has_extra) {
        // four threads per row, every fourth k each (all loads first, then one chain of multiply-adds), combined in
        // a fixed order
        const int r = tid >> 2, part = tid & 3, gm = (slot + i * ctas_per_blk) * TBM + r;
        const float *ar = lin + r * K + part;
        for (int x = 0; x < n_extra; ++x) {
          const float *bx = B + (size_t)(nblk * TBN + x) * K + part;
          float av[SK::KP_MAX / 4], bv[SK::KP_MAX / 4];
#pragma unroll
          for (int m = 0; m < SK::KP_MAX / 4; ++m) {
            const bool in = 4 * m + part < K;
            av[m] = in ? ar[4 * m] : 0.0f;
            bv[m] = in ? __ldg(bx + 4 * m) : 0.0f;
          }
          float acc = 0.0f;
#pragma unroll
          for (int m = 0; m < SK::KP_MAX / 4; ++m) acc = fmaf(av[m], bv[m], acc);
          acc += __shfl_xor_sync(0xffffffffu, acc, 1);
          acc += __shfl_xor_sync(0xffffffffu, acc, 2);
          if (part == 0 && gm < M) C[(size_t)gm * N + nblk * TBN + x] = acc;
        }
      }
      SK_STAMP(6 + 8 * i);
      {
        float v[SK::EPT];
#pragma unroll
        for (int j = 0; j < SK::EPT; ++j) {
          const int e = tid + SK::WORKERS * j;
          v[j] = e < tile_elems ? lin[e] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < SK::EPT; ++j) {
          const int e = tid + SK::WORKERS * j;
          if (e < tile_elems) {
            float h, l;
            split_tf32_rn(v[j], h, l);
            *reinterpret_cast<float *>(a_hi + off[j]) = h;
            *reinterpret_cast<float *>(a_lo + off[j]) = l;
          }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // this thread's writes -> tensor-core proxy
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ready);
      SK_STAMP(7 + 8 * i);
      if (i >= 1 && !*failed) store_tile(i - 1);   // while the tensor core multiplies tile i
    }
    if (nt > 0 && !*failed && !mbar_wait(bar_done, (uint32_t)((nt - 1) & 1))) *failed = 1;
    if (nt > 0 && !*failed) store_tile(nt - 1);
  } else if (lane == 0) {
    // ---- copy and MMA issue: one thread -------------------------------------------------------------------
    constexpr uint32_t ID = IDesc<true, true, TBN>::value;
    auto load_tile = [&](int i) {   // the CTA's i-th row tile -> linear buffer (rows past M keep stale values: never stored)
      const size_t a0 = (size_t)(slot + i * ctas_per_blk) * TBM * K, aend = (size_t)M * K;
      const size_t left = aend - a0;
      const uint32_t elems = left < (size_t)tile_elems ? (uint32_t)left : (uint32_t)tile_elems;
      const uint32_t bulk = (elems * 4u) & ~15u;
      for (uint32_t e = bulk / 4; e < elems; ++e) lin[e] = A[a0 + e];   // at most three floats of a ragged last tile
      mbar_expect_tx(bar_load, bulk);   // (release: the plain stores above are visible to whoever sees the phase)
      bulk_load(smem_u32(lin), A + a0, bulk, bar_load);
    };
    if (nt > 0) load_tile(0);
    for (int i = 0; i < nt; ++i) {
      if (*failed || !mbar_wait(bar_ready, (uint32_t)(i & 1))) {
        *failed = 1;
        break;
      }
      if (i + 1 < nt) load_tile(i + 1);   // every worker has read tile i out of the linear buffer
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t d = tmem_d + (uint32_t)((i & 1) * TBN);
      const uint32_t ah = smem_u32(a_hi), al = smem_u32(a_lo), bh = smem_u32(b_hi), bl = smem_u32(b_lo);
      for (int ks = 0; ks < ksteps; ++ks) {
        const uint32_t adv = ks * 2 * LBO_BYTES;   // 8 tf32 along k: two 16-byte chunks
        const uint64_t dah = make_desc<true>(ah + adv), dal = make_desc<true>(al + adv);
        const uint64_t dbh = make_desc<true>(bh + adv), dbl = make_desc<true>(bl + adv);
        mma_tf32(d, dal, dbh, ID, ks ? 1u : 0u);
        mma_tf32(d, dah, dbl, ID, 1u);
        mma_tf32(d, dah, dbh, ID, 1u);
      }
      commit_to(bar_done);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*failed && tid == 0) atomicExch(status, 202);
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)(2 * TBN)) : "memory");
  }
}

}  // namespace dgtc
