// Generated blocks: load and launch device code that the host's renderer emits for the elementwise
// blocks no recognised primitive covers (the CUDA counterpart of compiling the C renderer's output with
// clang and dlopen-ing it, Sources/DGen/Runtime.swift:291-311).  Two ways in:
//   dgc_module_load     a finished image (cubin for sm_100a, or NUL-terminated PTX),
//   dgc_module_compile  CUDA C source, compiled in process for sm_100a by NVRTC (loaded on first use;
//                       nothing links against it, so hosts that ship images never need it).
// Kernels are looked up by their extern "C" name and launched on the context stream.
#include <dlfcn.h>

#include <string>
#include <vector>

#include "common.cuh"

struct dgc_module {
  dgc_ctx *ctx;
  cudaLibrary_t lib;
  std::map<std::string, cudaKernel_t> kernels;
};

namespace {

// the few NVRTC entry points used, resolved at run time
struct Nvrtc {
  void *handle = nullptr;
  int (*create)(void **, const char *, const char *, int, const char *const *, const char *const *) = nullptr;
  int (*compile)(void *, int, const char *const *) = nullptr;
  int (*cubin_size)(void *, size_t *) = nullptr;
  int (*cubin)(void *, char *) = nullptr;
  int (*log_size)(void *, size_t *) = nullptr;
  int (*log)(void *, char *) = nullptr;
  int (*destroy)(void **) = nullptr;
  bool ok = false;
};

Nvrtc &nvrtc() {
  static Nvrtc n;
  if (n.handle || n.ok) return n;
  std::vector<std::string> names;
  if (const char *e = getenv("DGC_NVRTC_PATH")) names.push_back(e);
  for (const char *c : {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                        "/usr/local/cuda/lib64/libnvrtc.so"})
    names.push_back(c);
  for (auto &nm : names) {
    n.handle = dlopen(nm.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (n.handle) break;
  }
  if (!n.handle) return n;
#define SYM(field, name) *(void **)(&n.field) = dlsym(n.handle, name)
  SYM(create, "nvrtcCreateProgram");
  SYM(compile, "nvrtcCompileProgram");
  SYM(cubin_size, "nvrtcGetCUBINSize");
  SYM(cubin, "nvrtcGetCUBIN");
  SYM(log_size, "nvrtcGetProgramLogSize");
  SYM(log, "nvrtcGetProgramLog");
  SYM(destroy, "nvrtcDestroyProgram");
#undef SYM
  n.ok = n.create && n.compile && n.cubin_size && n.cubin && n.log_size && n.log && n.destroy;
  return n;
}

}  // namespace

DGC_EXPORT int32_t dgc_module_load(dgc_ctx *ctx, const void *image, uint64_t size, dgc_module **out) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, image && size > 0 && out, "null image or output");
  cudaLibrary_t lib = nullptr;
  cudaError_t e = cudaLibraryLoadData(&lib, image, nullptr, nullptr, 0, nullptr, nullptr, 0);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return dgc_fail(ctx, DGC_ERR_CUDA, "dgc_module_load: %s (the image must be a cubin for sm_100a or PTX text)",
                    cudaGetErrorString(e));
  }
  // loading is lazy by default: ask for the kernel count so that a bad image is refused here, with the
  // module handle never handed out, rather than at some later launch
  unsigned int count = 0;
  e = cudaLibraryGetKernelCount(&count, lib);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    cudaLibraryUnload(lib);
    return dgc_fail(ctx, DGC_ERR_INVALID, "dgc_module_load: the image holds no loadable kernel for this device (%s)",
                    e != cudaSuccess ? cudaGetErrorString(e) : "kernel count 0");
  }
  dgc_module *m = new dgc_module();
  m->ctx = ctx;
  m->lib = lib;
  *out = m;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_module_compile(dgc_ctx *ctx, const char *cuda_source, const char *name, dgc_module **out) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, cuda_source && out, "null source or output");
  Nvrtc &n = nvrtc();
  if (!n.ok) return dgc_fail(ctx, DGC_ERR_UNSUPPORTED, "dgc_module_compile: libnvrtc not found (set DGC_NVRTC_PATH)");
  void *prog = nullptr;
  if (n.create(&prog, cuda_source, name ? name : "dgen_block.cu", 0, nullptr, nullptr) != 0)
    return dgc_fail(ctx, DGC_ERR_CUDA, "nvrtcCreateProgram failed");
  // multiply-add contraction stays on, as in the reference's own build of generated code
  // (-ffp-contract=fast, Sources/DGen/DGenToolchainPolicy.swift:21-35)
  const char *opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo"};
  int rc = n.compile(prog, 3, opts);
  if (rc != 0) {
    size_t ls = 0;
    n.log_size(prog, &ls);
    std::string log(ls ? ls : 1, '\0');
    if (ls) n.log(prog, &log[0]);
    n.destroy(&prog);
    return dgc_fail(ctx, DGC_ERR_INVALID, "generated block does not compile: %.400s", log.c_str());
  }
  size_t cs = 0;
  n.cubin_size(prog, &cs);
  std::vector<char> image(cs);
  if (cs == 0 || n.cubin(prog, image.data()) != 0) {
    n.destroy(&prog);
    return dgc_fail(ctx, DGC_ERR_CUDA, "nvrtcGetCUBIN failed");
  }
  n.destroy(&prog);
  return dgc_module_load(ctx, image.data(), image.size(), out);
}

DGC_EXPORT int32_t dgc_module_unload(dgc_module *m) {
  if (!m) return DGC_ERR_INVALID;
  cudaStreamSynchronize(m->ctx->stream);
  cudaLibraryUnload(m->lib);
  delete m;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_launch(dgc_module *m, const char *kernel_name, const uint32_t grid[3], const uint32_t block[3],
                              uint32_t smem_bytes, void **args) {
  if (!m) return DGC_ERR_INVALID;
  dgc_ctx *ctx = m->ctx;
  DGC_REQUIRE(ctx, kernel_name && grid && block, "null argument");
  DGC_REQUIRE(ctx, grid[0] && grid[1] && grid[2] && block[0] && block[1] && block[2], "empty grid or block");
  DGC_REQUIRE(ctx, (uint64_t)block[0] * block[1] * block[2] <= 1024, "more than 1024 threads per block");
  auto it = m->kernels.find(kernel_name);
  if (it == m->kernels.end()) {
    cudaKernel_t k = nullptr;
    cudaError_t e = cudaLibraryGetKernel(&k, m->lib, kernel_name);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return dgc_fail(ctx, DGC_ERR_INVALID, "dgc_launch: no kernel '%s' in the module (%s)", kernel_name,
                      cudaGetErrorString(e));
    }
    it = m->kernels.emplace(kernel_name, k).first;
  }
  if (smem_bytes > 48 * 1024)
    DGC_CUDA(ctx, cudaFuncSetAttribute((const void *)it->second, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem_bytes));
  DGC_CUDA(ctx, cudaLaunchKernel((const void *)it->second, dim3(grid[0], grid[1], grid[2]),
                                 dim3(block[0], block[1], block[2]), args, smem_bytes, ctx->stream));
  ctx->launches++;
  return dgc_check_launch(ctx, kernel_name);
}
