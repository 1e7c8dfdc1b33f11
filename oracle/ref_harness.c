/*
 * Runs one reference-generated artefact (a shared object built by build_ref.sh from
 * toolchain/generated/hermetic/<name>.c of the reference tree) the way the reference's own
 * harness does (toolchain/harness/toolchain_harness.c:237-290): load, look up dgen_process_v1,
 * give it a caller-owned float arena, call it block by block.  TEST INFRASTRUCTURE.
 *
 * The four host services normally come from Apple Accelerate (vDSP_fft_zip, vDSP_zvma:
 * Sources/DGenHostSupport/DGenHostSupport.c:5-49), which does not exist here; they are supplied
 * by a plain radix-2 complex FFT (unnormalised both ways, like vDSP_fft_zip) and a complex
 * multiply-accumulate, so the artefact's own buffering, ring, hop-gating and overlap-add code is
 * what is exercised.
 */
#include <dlfcn.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

typedef void *FFTSetup;
typedef struct { uint32_t abi_version, struct_size; float sample_rate; uint32_t reserved; } Ctx;
typedef struct {
  uint32_t abi_version, struct_size;
  FFTSetup (*create)(uint32_t);
  void (*fwd)(FFTSetup, float *, float *, uint32_t);
  void (*inv)(FFTSetup, float *, float *, uint32_t);
  void (*mac)(const float *, const float *, const float *, const float *, float *, float *, uint32_t);
} Host;
typedef void (*ProcessFn)(const float *const *, float *const *, uint32_t, void *, const Ctx *, const Host *);

static void fft(float *re, float *im, int N, int inverse) {
  int j = 0;
  for (int i = 1; i < N; ++i) {
    int bit = N >> 1;
    for (; j & bit; bit >>= 1) j ^= bit;
    j ^= bit;
    if (i < j) { float t = re[i]; re[i] = re[j]; re[j] = t; t = im[i]; im[i] = im[j]; im[j] = t; }
  }
  for (int len = 2; len <= N; len <<= 1) {
    int half = len >> 1;
    for (int k = 0; k < half; ++k) {
      double ang = 2.0 * M_PI * k / len;
      float wr = (float)cos(ang), wi = (float)(inverse ? sin(ang) : -sin(ang));
      for (int i = k; i < N; i += len) {
        int jj = i + half;
        float tr = wr * re[jj] - wi * im[jj], ti = wr * im[jj] + wi * re[jj];
        re[jj] = re[i] - tr; im[jj] = im[i] - ti; re[i] += tr; im[i] += ti;
      }
    }
  }
}
static FFTSetup h_create(uint32_t l) { return (FFTSetup)(uintptr_t)(l + 1); }
static void h_fwd(FFTSetup s, float *re, float *im, uint32_t l) { (void)s; fft(re, im, 1 << l, 0); }
static void h_inv(FFTSetup s, float *re, float *im, uint32_t l) { (void)s; fft(re, im, 1 << l, 1); }
static void h_mac(const float *ar, const float *ai, const float *br, const float *bi, float *cr, float *ci,
                  uint32_t n) {
  for (uint32_t i = 0; i < n; ++i) {
    float r = ar[i] * br[i] - ai[i] * bi[i], m = ar[i] * bi[i] + ai[i] * br[i];
    cr[i] += r; ci[i] += m;
  }
}

/* Returns 0 on success.  memory: caller-initialised arena (persistent across blocks).
 * input may be NULL (instrument).  total frames = blocks * block_frames, block_frames % 4 == 0. */
int ref_run(const char *so_path, float *memory, const float *input, float *output, int blocks, int block_frames,
            float sample_rate) {
  void *h = dlopen(so_path, RTLD_NOW | RTLD_LOCAL);
  if (!h) { fprintf(stderr, "dlopen(%s): %s\n", so_path, dlerror()); return 1; }
  ProcessFn fn = (ProcessFn)dlsym(h, "dgen_process_v1");
  if (!fn) { dlclose(h); return 2; }
  Ctx ctx = {1u, sizeof(Ctx), sample_rate, 0};
  Host host = {1u, sizeof(Host), h_create, h_fwd, h_inv, h_mac};
  float zero_in[4096];
  memset(zero_in, 0, sizeof(zero_in));
  if (block_frames > 4096 && !input) { dlclose(h); return 3; }
  for (int b = 0; b < blocks; ++b) {
    const float *in0 = input ? input + (size_t)b * block_frames : zero_in;
    float *out0 = output + (size_t)b * block_frames;
    const float *ins[1] = {in0};
    float *outs[1] = {out0};
    fn(ins, outs, (uint32_t)block_frames, memory, &ctx, &host);
  }
  dlclose(h);
  return 0;
}
