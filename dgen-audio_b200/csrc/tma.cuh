// Tensor-map (TMA) tile loads of this GPU's own memory into shared memory, completion on an mbarrier with a
// bounded wait.  Every load is issued by one thread of a CTA for that CTA alone (plain loads, no fan-out to other CTAs).
//
// Used to stage the run of samples that the windows of one block cover (hop-gated buffer -> FFT): the copy engine
// fetches [rows = voices][columns = frames] boxes of the signal, frames before the start of the signal (negative
// coordinates) arrive as zeros, and no thread spends issue slots on addresses, bounds tests or the loads themselves.
// Rules the callers keep: the innermost coordinate is a multiple of 4 floats (16 bytes), the shared-memory
// destination is 128-byte aligned, the row stride of the tensor is a multiple of 16 bytes.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dgtma {

// ---- host: encode a 2-D float tensor map [rows][cols] (cols contiguous) with boxes of box_cols x 1 -------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// false when the driver entry point is missing or the tensor does not meet the alignment rules
inline bool make_map_2d(CUtensorMap *map, const float *base, uint64_t rows, uint64_t cols, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || (((uintptr_t)base) & 15) != 0 || (cols & 3) != 0 || box_cols == 0 || box_cols > 256 || (box_cols & 3) != 0)
    return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * sizeof(float)};
  const cuuint32_t box[2] = {box_cols, 1};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ---- device ------------------------------------------------------------------------------------------------
#ifdef __CUDACC__
constexpr uint32_t WAIT_LIMIT = 1u << 22;   // polls of the mbarrier before a wait gives up (tens of milliseconds)

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
  // make the initialised barrier visible to the asynchronous proxy (the copy engine)
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

// true when the phase with the given parity has completed; gives up after WAIT_LIMIT polls
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  const uint32_t a = smem_addr(bar);
  for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(a), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// one box of the map at (x = column, y = row) -> dst; completes `bytes of the box` on the barrier.
// x must be a multiple of 4 (16 bytes); it may be negative or past the end: those elements arrive as zeros.
__device__ __forceinline__ void load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_addr(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_addr(bar))
      : "memory");
}
#endif

}  // namespace dgtma
