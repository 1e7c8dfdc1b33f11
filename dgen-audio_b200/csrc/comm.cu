// Gradient exchange through the C ABI: one NCCL communicator per context, all-reduce (sum) in place on
// the context stream.  The training step's only data-path exchange is the all-reduce of the flat
// controller-gradient vector; a host without a Python runtime (the reference's host is Swift) gets it
// from here.  NCCL is resolved at run time (libnccl.so.2: the copy already loaded in the process if there
// is one), so the library has no link-time dependency on it and single-GPU hosts never load it.
// The unique id is created by rank 0 and handed to the other ranks by the host over any channel it has.
#include <dlfcn.h>

#include "common.cuh"

#include <cstring>

// layout of ncclUniqueId (a struct of 128 chars, passed by value to ncclCommInitRank)
struct Id128 {
  char internal[DGC_COMM_ID_BYTES];
};

namespace {

struct Nccl {
  void *handle = nullptr;
  int (*get_unique_id)(Id128 *) = nullptr;                                             // ncclGetUniqueId
  int (*comm_init_rank)(void **, int, Id128, int) = nullptr;                           // ncclCommInitRank
  int (*all_reduce)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
  int (*comm_destroy)(void *) = nullptr;
  const char *(*get_error_string)(int) = nullptr;
  bool ok = false;
};

Nccl &nccl() {
  static Nccl n;
  if (n.handle) return n;
  const char *names[] = {getenv("DGC_NCCL_PATH"), "libnccl.so.2", "libnccl.so"};
  for (const char *nm : names) {
    if (!nm) continue;
    n.handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
    if (n.handle) break;
  }
  if (!n.handle) return n;
#define SYM(field, name) *(void **)(&n.field) = dlsym(n.handle, name)
  SYM(get_unique_id, "ncclGetUniqueId");
  SYM(comm_init_rank, "ncclCommInitRank");
  SYM(all_reduce, "ncclAllReduce");
  SYM(comm_destroy, "ncclCommDestroy");
  SYM(get_error_string, "ncclGetErrorString");
#undef SYM
  n.ok = n.get_unique_id && n.comm_init_rank && n.all_reduce && n.comm_destroy;
  return n;
}

const char *nccl_err(Nccl &n, int rc) { return n.get_error_string ? n.get_error_string(rc) : "NCCL error"; }

}  // namespace

DGC_EXPORT int32_t dgc_comm_unique_id(uint8_t *id_out) {
  if (!id_out) return DGC_ERR_INVALID;
  Nccl &n = nccl();
  if (!n.ok) return DGC_ERR_UNSUPPORTED;
  Id128 id;
  if (n.get_unique_id(&id) != 0) return DGC_ERR_CUDA;
  memcpy(id_out, id.internal, DGC_COMM_ID_BYTES);
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_comm_init(dgc_ctx *ctx, int32_t world, int32_t rank, const uint8_t *id) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, id && world >= 1 && rank >= 0 && rank < world, "bad world / rank / id");
  DGC_REQUIRE(ctx, !ctx->comm, "the context already has a communicator");
  Nccl &n = nccl();
  if (!n.ok) return dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "dgc_comm_init: libnccl.so.2 not found (set DGC_NCCL_PATH)");
  DGC_CUDA(ctx, cudaSetDevice(ctx->device));
  Id128 uid;
  memcpy(uid.internal, id, DGC_COMM_ID_BYTES);
  void *comm = nullptr;
  int rc = n.comm_init_rank(&comm, world, uid, rank);
  if (rc != 0) return dgc_fail(ctx, DGC_ERR_CUDA, "ncclCommInitRank: %s", nccl_err(n, rc));
  ctx->comm = comm;
  ctx->comm_world = world;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_allreduce_sum(dgc_ctx *ctx, float *buf_dev, uint64_t n_floats) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, buf_dev || n_floats == 0, "null buffer");
  if (n_floats == 0) return DGC_OK;
  if (!ctx->comm) {
    // a context without a communicator is a world of one: the sum over ranks is the buffer itself
    return DGC_OK;
  }
  // The collective must not be part of a recorded step: a two-GPU run with the all-reduce inside the recording
  // never finished.  End the recording, exchange, record the update separately.
  DGC_REQUIRE(ctx, !ctx->capturing,
              "the gradient exchange cannot be recorded: end the recording (dgc_graph_end), exchange, and record "
              "the optimizer update as a second step");
  Nccl &n = nccl();
  // ncclFloat32 = 7, ncclSum = 0 (nccl.h enums ncclDataType_t / ncclRedOp_t, stable since NCCL 2.0)
  int rc = n.all_reduce(buf_dev, buf_dev, (size_t)n_floats, 7, 0, ctx->comm, ctx->stream);
  if (rc != 0) return dgc_fail(ctx, DGC_ERR_CUDA, "ncclAllReduce: %s", nccl_err(n, rc));
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_comm_destroy(dgc_ctx *ctx) {
  if (!ctx) return DGC_ERR_INVALID;
  if (!ctx->comm) return DGC_OK;
  cudaStreamSynchronize(ctx->stream);
  nccl().comm_destroy(ctx->comm);
  ctx->comm = nullptr;
  ctx->comm_world = 1;
  return DGC_OK;
}
