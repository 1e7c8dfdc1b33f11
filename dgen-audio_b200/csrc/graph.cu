// Step replay: record everything a host enqueues for one step on the context's stream once, then launch the
// recorded work with one call per step.
//
// The reference rebuilds and recompiles its graph and re-uploads every tensor on each training step
// (Sources/DGenLazy/Backward.swift:225, Sources/DGenLazy/Realize.swift:285-290, Sources/DGenLazy/LazyGraph.swift:171-234);
// with parameters, optimizer state and activations resident on the device the remaining per-step host cost is
// the launch sequence itself (about a hundred launches over three streams for the training step).  A CUDA graph
// replays that sequence, side-stream fork / join included, in one submission.
//
// Rules for the recorded region (checked where they can be):
//  * the context must be bound to a stream of its own or of the caller's, not the legacy default stream;
//  * every buffer a call may allocate (context scratch, cached tables, transposed-weight copies) must exist
//    already: run the step once before recording it;
//  * a call AFTER the recording that grows one of those buffers frees the addresses the recording holds: the
//    context counts such reallocations and dgc_graph_launch then refuses with DGC_ERR_INVALID ("record the step
//    again") instead of replaying into freed memory;
//  * values passed by value are frozen into the recording (sizes, the learning rate); anything that changes from
//    step to step must live in device memory -- inputs are refilled in place, the Adam step index is counted on
//    the device (dgc_adam_step_counted).
#include "common.cuh"

struct dgc_graph {
  dgc_ctx *ctx = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  uint64_t nodes = 0;
  int64_t launches = 0;   // launches the library counted while recording: added to the context's count per replay
  uint64_t generation = 0;  // the context's buffer generation when the recording ended
};

DGC_EXPORT int32_t dgc_graph_begin(dgc_ctx *ctx) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, ctx->stream != nullptr && ctx->stream != cudaStreamLegacy,
              "bind the context to a non-default stream before recording (dgc_ctx_set_stream)");
  DGC_REQUIRE(ctx, !ctx->capturing, "a recording is already in progress");
  // relaxed: other threads of the process (a data loader that allocates) must not invalidate the recording
  DGC_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
  ctx->capturing = true;
  ctx->capture_stream = ctx->stream;
  ctx->capture_launches0 = ctx->launches;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_graph_end(dgc_ctx *ctx, dgc_graph **out) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, out, "null pointer");
  DGC_REQUIRE(ctx, ctx->capturing, "no recording in progress");
  *out = nullptr;
  ctx->capturing = false;
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(ctx->capture_stream, &g);
  if (e != cudaSuccess || !g) {
    cudaGetLastError();
    return dgc_fail(ctx, DGC_ERR_CUDA, "the recording was invalidated (%s): a call inside it synchronised, allocated "
                                       "on first use, or used a stream that was not joined back",
                    cudaGetErrorString(e));
  }
  dgc_graph *r = new dgc_graph();
  r->ctx = ctx;
  r->graph = g;
  r->launches = ctx->launches - ctx->capture_launches0;
  r->generation = ctx->buffer_generation;
  size_t n = 0;
  cudaGraphGetNodes(g, nullptr, &n);
  r->nodes = n;
  e = cudaGraphInstantiate(&r->exec, g, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(g);
    delete r;
    return dgc_fail(ctx, DGC_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
  }
  *out = r;
  return DGC_OK;
}

DGC_EXPORT uint64_t dgc_graph_nodes(const dgc_graph *g) { return g ? g->nodes : 0; }

DGC_EXPORT int32_t dgc_graph_launch(dgc_ctx *ctx, dgc_graph *g) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, g && g->exec, "null graph");
  DGC_REQUIRE(ctx, g->ctx == ctx, "the graph was recorded on another context");
  DGC_REQUIRE(ctx, !ctx->capturing, "a recording is in progress");
  // A later call that needed more scratch freed and reallocated a context-owned buffer: the recording still
  // holds the old addresses and would read and write freed memory.  Nothing is launched.
  if (g->generation != ctx->buffer_generation)
    return dgc_fail(ctx, DGC_ERR_INVALID,
                    "dgc_graph_launch: a context buffer was reallocated after this step was recorded "
                    "(a later call needed more scratch): record the step again");
  DGC_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
  ctx->launches += g->launches;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_graph_destroy(dgc_graph *g) {
  if (!g) return DGC_OK;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
  return DGC_OK;
}
