// Shared declarations of libdgen_cuda: context object, error plumbing, launch helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <string>
#include <utility>

#include "../../include/dgen_cuda.h"

#define DGC_EXPORT extern "C" __attribute__((visibility("default")))

struct dgc_ctx {
  int device = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev_begin = nullptr, ev_end = nullptr, ev_sync = nullptr;
  int32_t *status_dev = nullptr;  // device status word: kernels report failures here
  unsigned int *ticket_dev = nullptr;  // last-block-done counter of the multi-block reductions (kept at 0)
  int64_t launches = 0;
  char err[512] = {0};
  int sm_count = 148;
  // context-owned scratch (grown on demand, never shrunk)
  float *scratch = nullptr;
  uint64_t scratch_floats = 0;
  // bumped whenever a context-owned device buffer (scratch, staging, transposed-operand copies) is freed or
  // reallocated: a recorded step holds raw pointers into those buffers and must be re-recorded afterwards
  uint64_t buffer_generation = 0;
  // cached data-independent tables
  std::map<std::pair<int, int>, float *> playheads;  // (F, T) -> device clock
  std::map<std::pair<int, int>, int *> row_ranges;   // (F, T) -> [F][4] frame ranges per control row
  std::map<std::pair<int, int>, float2 *> row_tables;  // (F, T) -> per frame (floor row as int bits, fraction)
  std::map<int, float *> hann_sym;                   // N -> symmetric Hann (spectral loss)
  std::map<int, float *> hann_per;                   // N -> periodic Hann (hann())
  std::map<int, float2 *> twiddles;                  // N -> exp(-2 pi i m / N), m < N
  double *loss_accum = nullptr;                      // 512 doubles: [0..64) results, [64..320) per-block sums
  float *wt_buf = nullptr;  // transposed copy of the current layer's weights (matmul forward)
  uint64_t wt_floats = 0;
  float *dzt_buf = nullptr;  // transposed copy of the current layer's output gradient (matmul backward)
  uint64_t dzt_floats = 0;
  // staging for the host-buffer composite entry points; uploads run on their own stream so that the
  // first kernels start while later inputs are still crossing PCIe
  cudaStream_t aux_stream = nullptr;   // second stream of the composite steps (noise branch beside the harmonic one)
  cudaEvent_t fork_ev = nullptr, join_ev = nullptr;
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t copy_ev[3] = {nullptr, nullptr, nullptr};
  float *stage_dev = nullptr;
  uint64_t stage_floats = 0;
  // two host-buffer steps in flight (plans.cu): per-slot input staging, upload events, end-of-step event
  float *pipe_in[2] = {nullptr, nullptr};
  uint64_t pipe_in_floats[2] = {0, 0};
  cudaEvent_t pipe_ev[2][3] = {{nullptr, nullptr, nullptr}, {nullptr, nullptr, nullptr}};
  cudaEvent_t pipe_done[2] = {nullptr, nullptr};
  bool pipe_used[2] = {false, false}, pipe_pending[2] = {false, false};
  // NCCL communicator of the gradient exchange (comm.cu); nullptr = a world of one
  void *comm = nullptr;
  int comm_world = 1;
  // spectral-loss backward: windows owned per block, chosen per (N, hop, H, B) so that the grid fills whole waves
  std::map<std::pair<std::pair<int, int>, std::pair<int, int>>, int> mss_bwd_owned;
  // matrix products issued per kernel family since the context was created (dgc_gemm_path_counts):
  // 0 SIMT register tiles, 1 tcgen05 generic-orientation kernel, 2 tcgen05 asynchronous pipeline, 3 the same with 128 x 256 tiles
  int64_t gemm_paths[4] = {0, 0, 0, 0};
  // step recording (graph.cu)
  bool capturing = false;
  cudaStream_t capture_stream = nullptr;   // the stream the recording started on (calls inside may rebind the context)
  int64_t capture_launches0 = 0;
};

// the caller-owned flat float arena (device memory) of dgc_arena_create
struct dgc_arena {
  dgc_ctx *ctx;
  float *ptr;
  uint64_t n;
  bool owned = true;   // false: the memory belongs to the caller (dgc_arena_wrap)
};

int32_t dgc_fail(dgc_ctx *ctx, int32_t code, const char *fmt, ...);
int32_t dgc_check_launch(dgc_ctx *ctx, const char *what);
// returns device pointer to at least n floats of context scratch (nullptr + error set on failure)
float *dgc_ctx_scratch(dgc_ctx *ctx, uint64_t nfloats);
// [F][4] ints: frames whose floor control row is r are [a,b) and [c,d) (second run: after the clock wrap)
const int *dgc_ctx_row_ranges(dgc_ctx *ctx, int F, int T);
// [T] float2: x = bits of the floor control row (int), y = lerp fraction of sampleRow at the cached clock
const float2 *dgc_ctx_row_table(dgc_ctx *ctx, int F, int T);
const float *dgc_ctx_hann_sym(dgc_ctx *ctx, int N);
const float *dgc_ctx_hann_per(dgc_ctx *ctx, int N);
// C[M][N] = A[M][K] * B[N][K]^T on the matmul path of gemm.cu
int32_t dgc_gemm_nt(dgc_ctx *ctx, const float *a, const float *b, int M, int N, int K, float *c);
// true when dgc_gemm_nt() runs this shape on its persistent short-reduction tensor-core kernel
bool dgc_gemm_nt_persistent(const dgc_ctx *ctx, const float *a, int M, int N, int K);
const float2 *dgc_ctx_twiddles(dgc_ctx *ctx, int N);
// dgc_mss_loss_fwd with the prediction given as the sum of two signals (pred_b may be null)
int32_t dgc_mss_loss_fwd_sum(dgc_ctx *ctx, const dgc_mss_params *p, const float *pred_dev, const float *pred_b_dev,
                             const float *target_dev, float *partial_dev, double *loss_dev);

#define DGC_CUDA(ctx, call)                                                                  \
  do {                                                                                       \
    cudaError_t e__ = (call);                                                                \
    if (e__ != cudaSuccess)                                                                  \
      return dgc_fail(ctx, e__ == cudaErrorMemoryAllocation ? DGC_ERR_OOM : DGC_ERR_CUDA,    \
                      "%s: %s", #call, cudaGetErrorString(e__));                             \
  } while (0)

#define DGC_REQUIRE(ctx, cond, msg)                            \
  do {                                                         \
    if (!(cond)) return dgc_fail(ctx, DGC_ERR_INVALID, "%s: %s", __func__, msg); \
  } while (0)

#define DGC_LAUNCHED(ctx, name)                     \
  do {                                              \
    (ctx)->launches++;                              \
    int32_t rc__ = dgc_check_launch(ctx, name);     \
    if (rc__ != DGC_OK) return rc__;                \
  } while (0)

static inline int dgc_div_up(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }
static inline bool dgc_is_pow2(int n) { return n > 0 && (n & (n - 1)) == 0; }
