// Block plans: the ordered list of blocks a host's matcher produced for one realize() / backward(), every buffer
// an offset into one arena, run by dgc_plan_run; and the harmonic+noise training step written as such a plan.
//
// The reference's scheduler partitions a graph into blocks (Sources/DGen/Blocks/BlockFormation.swift:5-85), its
// renderer emits one kernel per block over one flat memory (Sources/DGen/Renderer/CRenderer.swift:479-1307,
// Sources/DGen/Renderer/Renderer.swift:134-143) and the runtime calls them in order.  Here a block is either one of
// this library's primitives (the recognised patterns) or a generated kernel (blocks.cu), and the "call them in
// order" loop lives in the library, so a host hands over ONE description per graph and replays it per step.
#include "common.cuh"

#include <vector>

namespace {

__global__ void plan_add_kernel(const float *a, const float *__restrict__ b, size_t n, float *out) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __fadd_rn(a[i], b[i]);
}

struct Resolver {
  dgc_ctx *ctx;
  dgc_arena *arena;
  int step;
  bool bad = false;
  // pointer to `need` floats at offset off (nullptr for DGC_PLAN_NONE when optional)
  float *at(uint64_t off, uint64_t need, bool optional = false) {
    if (off == DGC_PLAN_NONE) {
      if (!optional) fail("a required buffer is absent");
      return nullptr;
    }
    if (off > arena->n || need > arena->n - off) {
      fail("a buffer reaches beyond the arena");
      return nullptr;
    }
    return arena->ptr + off;
  }
  void fail(const char *what) {
    if (!bad) dgc_fail(ctx, DGC_ERR_INVALID, "dgc_plan_run: step %d: %s", step, what);
    bad = true;
  }
};

dgc_mss_params mss_of(const dgc_plan_step &s) {
  dgc_mss_params m;
  memset(&m, 0, sizeof(m));
  m.B = s.i[0];
  m.T = s.i[1];
  m.nscales = s.i[2];
  m.hop_div = s.i[3];
  for (int k = 0; k < DGC_MSS_MAX_SCALES && k < m.nscales; ++k) m.sizes[k] = s.i[4 + k];
  m.w_lin = s.f[0];
  m.w_log = s.f[1];
  return m;
}

}  // namespace

DGC_EXPORT int32_t dgc_plan_run(dgc_ctx *ctx, dgc_arena *arena, const dgc_plan *plan, int32_t first, int32_t count) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, arena && plan && plan->steps && arena->ctx == ctx, "null plan / arena, or an arena of another context");
  DGC_REQUIRE(ctx, first >= 0 && first <= plan->n_steps, "first step out of range");
  const int last = count < 0 ? plan->n_steps : first + count;
  DGC_REQUIRE(ctx, last <= plan->n_steps, "step range out of range");
  if (!ctx->aux_stream) {
    DGC_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->aux_stream, cudaStreamNonBlocking));
    DGC_CUDA(ctx, cudaEventCreateWithFlags(&ctx->fork_ev, cudaEventDisableTiming));
    DGC_CUDA(ctx, cudaEventCreateWithFlags(&ctx->join_ev, cudaEventDisableTiming));
  }
  cudaStream_t main_stream = ctx->stream;
  bool forked = false;
  int32_t rc = DGC_OK;
  Resolver R{ctx, arena, 0};
  auto join = [&]() {
    if (forked) {
      cudaEventRecord(ctx->join_ev, ctx->aux_stream);
      cudaStreamWaitEvent(main_stream, ctx->join_ev, 0);
      forked = false;
    }
  };
  for (int k = first; k < last && rc == DGC_OK; ++k) {
    const dgc_plan_step &s = plan->steps[k];
    R.step = k;
    if (s.stream == 1 && !forked && s.op != DGC_PLAN_FORK) {
      rc = dgc_fail(ctx, DGC_ERR_INVALID, "dgc_plan_run: step %d runs on the side stream before a FORK", k);
      break;
    }
    ctx->stream = s.stream == 1 ? ctx->aux_stream : main_stream;
    const uint64_t *a = s.a;
    const int32_t *i = s.i;
    const float *f = s.f;
    switch (s.op) {
      case DGC_PLAN_FORK:
        if (!forked) {
          if (cudaEventRecord(ctx->fork_ev, main_stream) != cudaSuccess ||
              cudaStreamWaitEvent(ctx->aux_stream, ctx->fork_ev, 0) != cudaSuccess)
            rc = dgc_fail(ctx, DGC_ERR_CUDA, "dgc_plan_run: step %d: fork failed", k);
          forked = true;
        }
        break;
      case DGC_PLAN_JOIN:
        join();
        break;
      case DGC_PLAN_OSC_BANK_CONST: {
        const float *fq = R.at(a[0], i[0]), *am = R.at(a[1], i[0]);
        float *out = R.at(a[2], i[1]);
        if (!R.bad) rc = dgc_osc_bank_const(ctx, fq, am, i[0], i[1], f[0], i[2], out);
      } break;
      case DGC_PLAN_HARMONIC_RENDER: {
        dgc_harmonic_params p{i[0], i[1], i[2], i[3], f[0], f[1], i[4], i[5]};
        const uint64_t fb = (uint64_t)p.F * p.B, bt = (uint64_t)p.B * p.T;
        const float *f0 = R.at(a[0], fb), *uv = R.at(a[1], fb), *amps = R.at(a[2], fb * p.K), *gain = R.at(a[3], fb);
        float *scr = R.at(a[4], dgc_harmonic_scratch_floats(&p), true), *out = R.at(a[5], bt);
        if (!R.bad) rc = dgc_harmonic_render(ctx, &p, f0, uv, amps, gain, scr, out);
      } break;
      case DGC_PLAN_BANDS_TO_TAPS: {
        const float *bands = R.at(a[0], (uint64_t)i[0] * i[1]), *w = R.at(a[1], (uint64_t)i[2] * i[1]);
        float *taps = R.at(a[2], (uint64_t)i[0] * i[2]);
        if (!R.bad) rc = dgc_bands_to_taps(ctx, bands, w, i[0], i[1], i[2], taps);
      } break;
      case DGC_PLAN_FIR_NOISE: {
        dgc_fir_params p{i[0], i[1], i[2], i[3], f[0], i[4]};
        const uint64_t fb = (uint64_t)p.F * p.B, bt = (uint64_t)p.B * p.T;
        const float *noise = R.at(a[0], bt), *taps = R.at(a[1], fb * p.taps), *ng = R.at(a[2], fb);
        float *out = R.at(a[3], bt);
        if (!R.bad) rc = dgc_fir_noise(ctx, &p, noise, taps, ng, out);
      } break;
      case DGC_PLAN_ADD: {
        const uint64_t n = a[3];
        const float *x = R.at(a[0], n), *y = R.at(a[1], n);
        float *out = R.at(a[2], n);
        if (!R.bad && n > 0) {
          plan_add_kernel<<<dgc_div_up((int64_t)n, 256), 256, 0, ctx->stream>>>(x, y, n, out);
          ctx->launches++;
          rc = dgc_check_launch(ctx, "plan_add");
        }
      } break;
      case DGC_PLAN_COPY: {
        const uint64_t n = a[2];
        const float *src = R.at(a[0], n);
        float *dst = R.at(a[1], n);
        if (!R.bad && n > 0 &&
            cudaMemcpyAsync(dst, src, n * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream) != cudaSuccess)
          rc = dgc_fail(ctx, DGC_ERR_CUDA, "dgc_plan_run: step %d: copy failed", k);
      } break;
      case DGC_PLAN_ONEPOLE: {
        const uint64_t bt = (uint64_t)i[0] * i[1];
        const float *x = R.at(a[0], bt);
        float *y = R.at(a[1], bt), *st = R.at(a[2], i[0], true);
        if (!R.bad) rc = dgc_onepole_fwd_state(ctx, x, i[0], i[1], f[0], st, y);
      } break;
      case DGC_PLAN_BIQUAD_FWD: {
        dgc_biquad_params p{i[0], i[1], i[2], f[0], f[1]};
        const uint64_t bt = (uint64_t)p.B * p.T;
        const float *x = R.at(a[0], bt), *cut = R.at(a[1], p.L), *q = R.at(a[2], p.L);
        float *scr = R.at(a[3], dgc_biquad_scratch_floats(&p, 0), true), *st = R.at(a[4], (uint64_t)p.B * 4 * p.L, true);
        float *y = R.at(a[5], bt * p.L);
        if (!R.bad) rc = dgc_biquad_fwd_state(ctx, &p, x, cut, q, scr, st, y);
      } break;
      case DGC_PLAN_BIQUAD_MSE_BWD: {
        dgc_biquad_params p{i[0], i[1], i[2], f[0], f[1]};
        const uint64_t bt = (uint64_t)p.B * p.T;
        const float *x = R.at(a[0], bt), *cut = R.at(a[1], p.L), *q = R.at(a[2], p.L), *y = R.at(a[3], bt * p.L),
                    *tg = R.at(a[4], bt * p.L);
        float *scr = R.at(a[5], dgc_biquad_scratch_floats(&p, 1), true), *gc = R.at(a[6], p.L), *gq = R.at(a[7], p.L);
        float *loss = R.at(a[8], 2);
        if (!R.bad && (a[8] & 1)) R.fail("a double must sit at an even offset");
        if (!R.bad) rc = dgc_biquad_mse_bwd(ctx, &p, x, cut, q, y, tg, f[2], scr, gc, gq, reinterpret_cast<double *>(loss));
      } break;
      case DGC_PLAN_STFT_MAG: {
        const int V = i[0], T = i[1], N = i[2], hop = i[3];
        const uint64_t H = hop > 0 ? (uint64_t)dgc_div_up(T, hop) : 0;
        const float *x = R.at(a[0], (uint64_t)V * T), *win = R.at(a[1], N, true);
        float *mags = R.at(a[2], (uint64_t)V * H * (N / 2 + 1));
        if (!R.bad) rc = dgc_stft_mag(ctx, x, V, T, N, hop, win, mags);
      } break;
      case DGC_PLAN_PARTCONV: {
        const int V = i[0], T = i[1], irl = i[2], N = i[3], hop = i[4];
        const float *x = R.at(a[0], (uint64_t)V * T), *ir = R.at(a[1], irl);
        float *scr = R.at(a[2], dgc_partconv_scratch_floats(V, T, irl, N, hop), true), *out = R.at(a[3], (uint64_t)V * T);
        if (!R.bad) rc = dgc_partconv(ctx, x, V, T, ir, irl, N, hop, f[0], scr, i[5], out);
      } break;
      case DGC_PLAN_PARTCONV_BWD: {
        const int V = i[0], T = i[1], irl = i[2], N = i[3], hop = i[4];
        const float *x = R.at(a[0], (uint64_t)V * T), *ir = R.at(a[1], irl), *go = R.at(a[2], (uint64_t)V * T);
        float *scr = R.at(a[3], dgc_partconv_bwd_scratch_floats(V, T, irl, N, hop), true);
        float *gx = R.at(a[4], (uint64_t)V * T, true), *gir = R.at(a[5], irl, true);
        if (!R.bad) rc = dgc_partconv_bwd(ctx, x, V, T, ir, irl, N, hop, f[0], go, scr, i[5], gx, gir);
      } break;
      case DGC_PLAN_MSS_LOSS_FWD: {
        const dgc_mss_params m = mss_of(s);
        const uint64_t bt = (uint64_t)m.B * m.T;
        const float *pred = R.at(a[0], bt), *tg = R.at(a[1], bt);
        float *part = R.at(a[2], dgc_mss_partial_floats(&m), true), *loss = R.at(a[3], 2);
        if (!R.bad && (a[3] & 1)) R.fail("a double must sit at an even offset");
        if (!R.bad) rc = dgc_mss_loss_fwd(ctx, &m, pred, tg, part, reinterpret_cast<double *>(loss));
      } break;
      case DGC_PLAN_MSS_LOSS_BWD: {
        const dgc_mss_params m = mss_of(s);
        const uint64_t bt = (uint64_t)m.B * m.T;
        const float *pred = R.at(a[0], bt), *tg = R.at(a[1], bt);
        float *g = R.at(a[2], bt);
        if (!R.bad) rc = dgc_mss_loss_bwd(ctx, &m, pred, tg, f[2], g);
      } break;
      case DGC_PLAN_LINEAR_FWD: {
        const uint64_t M = i[0], K = i[1], N = i[2];
        const float *A = R.at(a[0], M * K), *W = R.at(a[1], K * N), *bias = R.at(a[2], N, true);
        float *Cm = R.at(a[3], M * N), *Ct = R.at(a[4], M * N, true);
        if (!R.bad) rc = dgc_linear_fwd(ctx, A, W, bias, i[0], i[1], i[2], i[3], Cm, Ct);
      } break;
      case DGC_PLAN_LINEAR_BWD: {
        const uint64_t M = i[0], K = i[1], N = i[2];
        const float *A = R.at(a[0], M * K), *W = R.at(a[1], K * N), *Cm = R.at(a[2], M * N), *dC = R.at(a[3], M * N);
        float *dZ = R.at(a[4], M * N), *dA = R.at(a[5], M * K, true), *dW = R.at(a[6], K * N), *db = R.at(a[7], N, true);
        const float *At = R.at(a[8], M * K, true);
        if (!R.bad) rc = dgc_linear_bwd(ctx, A, W, Cm, dC, i[0], i[1], i[2], i[3], dZ, dA, dW, db, At);
      } break;
      case DGC_PLAN_HEADS_FWD: {
        const uint64_t M = i[0], K = i[1], NB = i[2];
        const float *z = R.at(a[0], M * (K + NB));
        float *amps = R.at(a[1], M * K), *bands = R.at(a[2], M * NB);
        if (!R.bad) rc = dgc_hn_heads_fwd(ctx, z, i[0], i[1], i[2], amps, bands);
      } break;
      case DGC_PLAN_HEADS_BWD: {
        const uint64_t M = i[0], K = i[1], NB = i[2];
        const float *z = R.at(a[0], M * (K + NB)), *ga = R.at(a[1], M * K), *gb = R.at(a[2], M * NB);
        float *gz = R.at(a[3], M * (K + NB));
        if (!R.bad) rc = dgc_hn_heads_bwd(ctx, z, ga, gb, i[0], i[1], i[2], gz);
      } break;
      case DGC_PLAN_HARMONIC_BWD: {
        dgc_harmonic_params p{i[0], i[1], i[2], i[3], f[0], f[1], i[4], 0};
        const uint64_t fb = (uint64_t)p.F * p.B, bt = (uint64_t)p.B * p.T;
        const float *f0 = R.at(a[0], fb), *uv = R.at(a[1], fb), *amps = R.at(a[2], fb * p.K), *gain = R.at(a[3], fb),
                    *ga = R.at(a[4], bt);
        float *scr = R.at(a[5], dgc_harmonic_bwd_scratch_floats(&p), i[5] == 0), *g = R.at(a[6], fb * p.K);
        if (!R.bad)
          rc = i[5] ? dgc_harmonic_render_bwd_prepared(ctx, &p, f0, uv, amps, gain, ga, scr, g)
                    : dgc_harmonic_render_bwd(ctx, &p, f0, uv, amps, gain, ga, scr, g);
      } break;
      case DGC_PLAN_FIR_BWD: {
        dgc_fir_params p{i[0], i[1], i[2], i[3], f[0], 0};
        const uint64_t fb = (uint64_t)p.F * p.B, bt = (uint64_t)p.B * p.T;
        const float *noise = R.at(a[0], bt), *ng = R.at(a[1], fb), *ga = R.at(a[2], bt);
        float *g = R.at(a[3], fb * p.taps);
        if (!R.bad) rc = dgc_fir_noise_bwd(ctx, &p, noise, ng, ga, g);
      } break;
      case DGC_PLAN_ALLREDUCE: {
        float *buf = R.at(a[0], a[1]);
        if (!R.bad) rc = dgc_allreduce_sum(ctx, buf, a[1]);
      } break;
      case DGC_PLAN_ADAM: {
        const uint64_t n = a[6];
        float *th = R.at(a[0], n), *g = R.at(a[1], n), *m = R.at(a[2], n), *v = R.at(a[3], n);
        float *t = R.at(a[4], 1), *corr = R.at(a[5], 2);
        if (!R.bad) rc = dgc_adam_step_counted(ctx, th, g, m, v, n, reinterpret_cast<int32_t *>(t), corr, f[0], f[1], f[2], f[3]);
      } break;
      case DGC_PLAN_SANITIZE: {
        const float *in = R.at(a[0], a[2]);
        float *out = R.at(a[1], a[2]);
        if (!R.bad) rc = dgc_sanitize(ctx, in, a[2], out);
      } break;
      case DGC_PLAN_BLOCK: {
        if (!plan->modules || !plan->kernels || i[0] < 0 || i[0] >= plan->n_kernels || !plan->modules[i[0]] ||
            !plan->kernels[i[0]]) {
          R.fail("no generated kernel with that index");
          break;
        }
        float *mem = arena->ptr;
        int c0 = i[2], c1 = i[3];
        void *args_e[] = {&mem, &c0};
        void *args_s[] = {&mem, &c0, &c1};
        const int threads = 128;
        const int work = i[1] == 0 ? c0 : c1;   // one thread per index (elementwise) or per lane (sequential)
        if (work <= 0) break;
        const uint32_t grid[3] = {(uint32_t)dgc_div_up(work, threads), 1, 1}, block[3] = {(uint32_t)threads, 1, 1};
        rc = dgc_launch(plan->modules[i[0]], plan->kernels[i[0]], grid, block, 0, i[1] == 0 ? args_e : args_s);
      } break;
      default:
        R.fail("unknown op");
    }
    if (R.bad) rc = DGC_ERR_INVALID;
    else if (rc != DGC_OK) {
      // keep the primitive's message, say which step it was
      char msg[sizeof(ctx->err)];
      snprintf(msg, sizeof(msg), "%s", ctx->err);
      dgc_fail(ctx, rc, "dgc_plan_run: step %d: %.400s", k, msg);
    }
  }
  ctx->stream = main_stream;
  join();
  return rc;
}

// ---------------------------------------------------------------------------------------------------------
// The harmonic+noise training step as a plan
// ---------------------------------------------------------------------------------------------------------
namespace {

struct Layouter {
  uint64_t used = 0;
  uint64_t take(uint64_t n) {
    const uint64_t off = used;
    used += (n + 63) & ~63ull;   // every buffer 256-byte aligned
    return off;
  }
};

dgc_plan_step mk(int op, int stream = 0) {
  dgc_plan_step s;
  memset(&s, 0, sizeof(s));
  s.op = op;
  s.stream = stream;
  for (auto &v : s.a) v = DGC_PLAN_NONE;
  return s;
}

void put_mss(dgc_plan_step &s, const dgc_mss_params &m, int B, int T) {
  s.i[0] = B;
  s.i[1] = T;
  s.i[2] = m.nscales;
  s.i[3] = m.hop_div;
  for (int k = 0; k < DGC_MSS_MAX_SCALES; ++k) s.i[4 + k] = k < m.nscales ? m.sizes[k] : 0;
  s.f[0] = m.w_lin;
  s.f[1] = m.w_log;
}

}  // namespace

DGC_EXPORT int32_t dgc_hn_train_plan(const dgc_hn_train_config *c, dgc_hn_train_layout *lay, dgc_plan_step *steps,
                                     int32_t cap) {
  if (!c || !lay) return DGC_ERR_INVALID;
  if (c->B <= 0 || c->T <= 0 || c->K <= 0 || c->F <= 0 || c->nbands <= 0 || c->taps <= 0 || c->in_features <= 0 ||
      c->hidden <= 0 || c->n_trunk < 1 || c->n_trunk > 8 || c->ir_len <= 0 || c->conv_n <= 0 || c->conv_hop <= 0 ||
      c->mss.nscales <= 0 || c->mss.nscales > DGC_MSS_MAX_SCALES || c->global_voices < c->B)
    return DGC_ERR_INVALID;
  const int B = c->B, T = c->T, K = c->K, F = c->F, NB = c->nbands, NT = c->taps, H = c->hidden, NL = c->n_trunk;
  const uint64_t M = (uint64_t)F * B, BT = (uint64_t)B * T, FB = M, OUT = (uint64_t)K + NB;
  Layouter L;
  // ---- parameters: W0 b0 .. W(NL-1) b(NL-1) Wh bh ir, one flat vector; gradient and Adam moments alike
  std::vector<uint64_t> w_off(NL + 1), b_off(NL + 1);
  uint64_t np = 0;
  for (int l = 0; l <= NL; ++l) {
    const uint64_t in = l == 0 ? c->in_features : H, out = l == NL ? OUT : H;
    w_off[l] = np;
    np += in * out;
    b_off[l] = np;
    np += out;
  }
  const uint64_t ir_off = np;
  np += c->ir_len;
  memset(lay, 0, sizeof(*lay));
  lay->n_params = np;
  lay->params = L.take(np);
  lay->grads = L.take(np);
  lay->adam_m = L.take(np);
  lay->adam_v = L.take(np);
  lay->adam_t = L.take(1);
  lay->adam_corr = L.take(2);
  lay->x = L.take(M * c->in_features);
  lay->f0 = L.take(FB);
  lay->uv = L.take(FB);
  lay->gain = L.take(FB);
  lay->noise_gain = L.take(FB);
  lay->noise = L.take(BT);
  lay->w_fs = L.take((uint64_t)NT * NB);
  lay->target = L.take(BT);
  lay->loss = L.take(2);
  lay->audio = L.take(BT);
  // ---- activations and work buffers
  std::vector<uint64_t> act(NL), act_t(NL), dact(NL), dz(NL);
  for (int l = 0; l < NL; ++l) {
    act[l] = L.take(M * H);
    act_t[l] = L.take(M * H);
    dact[l] = L.take(M * H);
    dz[l] = L.take(M * H);
  }
  const uint64_t z = L.take(M * OUT), dz_head = L.take(M * OUT), head_dz = L.take(M * OUT);
  const uint64_t amps = L.take(M * K), bands = L.take(M * NB), g_amps = L.take(M * K), g_bands = L.take(M * NB);
  const uint64_t taps_tab = L.take(M * NT), g_taps = L.take(M * NT);
  const uint64_t dry = L.take(BT), noise_out = L.take(BT), g_out = L.take(BT);
  dgc_harmonic_params hp{B, T, K, F, c->sample_rate, 1.0f, c->phase_mode, 0};
  const uint64_t h_scratch = L.take(dgc_harmonic_bwd_scratch_floats(&hp) + 64);
  lay->total_floats = L.used;

  std::vector<dgc_plan_step> S;
  auto P = [&](uint64_t off) { return lay->params + off; };
  auto G = [&](uint64_t off) { return lay->grads + off; };
  // ---- forward: controller
  for (int l = 0; l <= NL; ++l) {
    dgc_plan_step s = mk(DGC_PLAN_LINEAR_FWD);
    s.a[0] = l == 0 ? lay->x : act[l - 1];
    s.a[1] = P(w_off[l]);
    s.a[2] = P(b_off[l]);
    s.a[3] = l == NL ? z : act[l];
    s.a[4] = l == NL ? DGC_PLAN_NONE : act_t[l];   // trunk activations are also kept transposed for the weight gradients
    s.i[0] = (int32_t)M;
    s.i[1] = l == 0 ? c->in_features : H;
    s.i[2] = l == NL ? (int32_t)OUT : H;
    s.i[3] = l == NL ? 0 : 1;
    S.push_back(s);
  }
  {
    dgc_plan_step s = mk(DGC_PLAN_HEADS_FWD);
    s.a[0] = z; s.a[1] = amps; s.a[2] = bands;
    s.i[0] = (int32_t)M; s.i[1] = K; s.i[2] = NB;
    S.push_back(s);
  }
  // ---- forward: the noise branch beside the harmonic branch
  S.push_back(mk(DGC_PLAN_FORK));
  {
    dgc_plan_step s = mk(DGC_PLAN_BANDS_TO_TAPS, 1);
    s.a[0] = bands; s.a[1] = lay->w_fs; s.a[2] = taps_tab;
    s.i[0] = (int32_t)M; s.i[1] = NB; s.i[2] = NT;
    S.push_back(s);
    s = mk(DGC_PLAN_FIR_NOISE, 1);
    s.a[0] = lay->noise; s.a[1] = taps_tab; s.a[2] = lay->noise_gain; s.a[3] = noise_out;
    s.i[0] = B; s.i[1] = T; s.i[2] = F; s.i[3] = NT; s.i[4] = 0;
    s.f[0] = 0.12f;
    S.push_back(s);
    s = mk(DGC_PLAN_HARMONIC_RENDER);
    s.a[0] = lay->f0; s.a[1] = lay->uv; s.a[2] = amps; s.a[3] = lay->gain; s.a[4] = h_scratch; s.a[5] = dry;
    s.i[0] = B; s.i[1] = T; s.i[2] = K; s.i[3] = F; s.i[4] = c->phase_mode; s.i[5] = 0;
    s.f[0] = c->sample_rate; s.f[1] = 1.0f;
    S.push_back(s);
  }
  S.push_back(mk(DGC_PLAN_JOIN));
  {
    dgc_plan_step s = mk(DGC_PLAN_ADD);
    s.a[0] = dry; s.a[1] = noise_out; s.a[2] = dry; s.a[3] = BT;
    S.push_back(s);
    s = mk(DGC_PLAN_COPY);
    s.a[0] = dry; s.a[1] = lay->audio; s.a[2] = BT;
    S.push_back(s);
    s = mk(DGC_PLAN_PARTCONV);   // out = dry + reverb(dry)
    s.a[0] = dry; s.a[1] = P(ir_off); s.a[3] = lay->audio;
    s.i[0] = B; s.i[1] = T; s.i[2] = c->ir_len; s.i[3] = c->conv_n; s.i[4] = c->conv_hop; s.i[5] = 1;
    s.f[0] = 1.0f;
    S.push_back(s);
    s = mk(DGC_PLAN_MSS_LOSS_FWD);
    s.a[0] = lay->audio; s.a[1] = lay->target; s.a[3] = lay->loss;
    put_mss(s, c->mss, B, T);
    S.push_back(s);
  }
  // ---- backward
  {
    dgc_plan_step s = mk(DGC_PLAN_MSS_LOSS_BWD);
    s.a[0] = lay->audio; s.a[1] = lay->target; s.a[2] = g_out;
    put_mss(s, c->mss, B, T);
    s.f[2] = (float)B / (float)c->global_voices;   // local share of the global-batch mean
    S.push_back(s);
    s = mk(DGC_PLAN_PARTCONV_BWD);   // g_dry = g_out + A(ir)^T g_out, in place; g_ir
    s.a[0] = dry; s.a[1] = P(ir_off); s.a[2] = g_out; s.a[4] = g_out; s.a[5] = G(ir_off);
    s.i[0] = B; s.i[1] = T; s.i[2] = c->ir_len; s.i[3] = c->conv_n; s.i[4] = c->conv_hop; s.i[5] = 1;
    s.f[0] = 1.0f;
    S.push_back(s);
  }
  S.push_back(mk(DGC_PLAN_FORK));
  {
    dgc_plan_step s = mk(DGC_PLAN_FIR_BWD, 1);
    s.a[0] = lay->noise; s.a[1] = lay->noise_gain; s.a[2] = g_out; s.a[3] = g_taps;
    s.i[0] = B; s.i[1] = T; s.i[2] = F; s.i[3] = NT;
    s.f[0] = 0.12f;
    S.push_back(s);
    s = mk(DGC_PLAN_LINEAR_FWD, 1);   // g_bands = g_taps Wfs
    s.a[0] = g_taps; s.a[1] = lay->w_fs; s.a[3] = g_bands;
    s.i[0] = (int32_t)M; s.i[1] = NT; s.i[2] = NB; s.i[3] = 0;
    S.push_back(s);
    s = mk(DGC_PLAN_HARMONIC_BWD);    // walks the phases the forward left in its scratch
    s.a[0] = lay->f0; s.a[1] = lay->uv; s.a[2] = amps; s.a[3] = lay->gain; s.a[4] = g_out; s.a[5] = h_scratch; s.a[6] = g_amps;
    s.i[0] = B; s.i[1] = T; s.i[2] = K; s.i[3] = F; s.i[4] = c->phase_mode; s.i[5] = 1;
    s.f[0] = c->sample_rate; s.f[1] = 1.0f;
    S.push_back(s);
  }
  S.push_back(mk(DGC_PLAN_JOIN));
  {
    dgc_plan_step s = mk(DGC_PLAN_HEADS_BWD);
    s.a[0] = z; s.a[1] = g_amps; s.a[2] = g_bands; s.a[3] = dz_head;
    s.i[0] = (int32_t)M; s.i[1] = K; s.i[2] = NB;
    S.push_back(s);
  }
  for (int l = NL; l >= 0; --l) {
    dgc_plan_step s = mk(DGC_PLAN_LINEAR_BWD);
    s.a[0] = l == 0 ? lay->x : act[l - 1];
    s.a[1] = P(w_off[l]);
    s.a[2] = l == NL ? z : act[l];
    s.a[3] = l == NL ? dz_head : dact[l];
    s.a[4] = l == NL ? head_dz : dz[l];
    s.a[5] = l > 0 ? dact[l - 1] : DGC_PLAN_NONE;
    s.a[6] = G(w_off[l]);
    s.a[7] = G(b_off[l]);
    s.a[8] = l > 0 ? act_t[l - 1] : DGC_PLAN_NONE;
    s.i[0] = (int32_t)M;
    s.i[1] = l == 0 ? c->in_features : H;
    s.i[2] = l == NL ? (int32_t)OUT : H;
    s.i[3] = l == NL ? 0 : 1;
    S.push_back(s);
  }
  lay->n_forward_backward = (int32_t)S.size();
  {
    dgc_plan_step s = mk(DGC_PLAN_ALLREDUCE);
    s.a[0] = lay->grads; s.a[1] = np;
    S.push_back(s);
    s = mk(DGC_PLAN_ADAM);
    s.a[0] = lay->params; s.a[1] = lay->grads; s.a[2] = lay->adam_m; s.a[3] = lay->adam_v; s.a[4] = lay->adam_t;
    s.a[5] = lay->adam_corr; s.a[6] = np;
    s.f[0] = c->lr; s.f[1] = c->beta1; s.f[2] = c->beta2; s.f[3] = c->eps;
    S.push_back(s);
  }
  lay->n_steps = (int32_t)S.size();
  if (!steps) return DGC_OK;
  if (cap < lay->n_steps) return DGC_ERR_INVALID;
  memcpy(steps, S.data(), S.size() * sizeof(dgc_plan_step));
  return DGC_OK;
}
