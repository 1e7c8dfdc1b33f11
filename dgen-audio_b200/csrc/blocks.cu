// Emitter for the elementwise blocks that no recognised primitive covers: a block is a short SSA program
// over arena cells, one thread per (frame, element) index, rendered to CUDA C with the SAME scalar
// expressions the reference's C renderer writes for each op (Sources/DGen/Renderer/CRenderer.swift:484-1040,
// scalar branch of every case; the frame loop `for (int i = 0; i < frameCount; i++)` becomes the thread
// index), then compiled for sm_100a through dgc_module_compile.  The Swift-side renderer that walks the
// reference's UOps would produce exactly this op list; it is host code of the reference and not part of
// this library.
//
// Blocks that read and write state cells (history feedback, phasor, latch: the reference's SEQUENTIAL blocks,
// Sources/DGen/Blocks/FeedbackAnalysis.swift:357-365) are emitted in a second form: one thread per tensor lane,
// the frame loop inside the thread in frame order, every state cell of the lane held in a register across the
// loop (loaded before, stored after).  Lanes are independent in the reference too (tensor history cells are
// per element, Sources/DGen/HigherOps.swift:408-420), so this is the same computation with the lane loop
// turned into the grid.
#include <cstdio>
#include <string>
#include <vector>

#include "common.cuh"

namespace {

struct Emit {
  std::string s;
  void line(const std::string &l) { s += "  " + l + "\n"; }
};

std::string fl(float v) {
  char b[64];
  if (v != v) return "__int_as_float(0x7fc00000)";
  if (v > 3.4e38f) return "__int_as_float(0x7f800000)";
  if (v < -3.4e38f) return "__int_as_float(0xff800000)";
  snprintf(b, sizeof b, "%.9gf", (double)v);
  std::string r(b);
  // "1f" is not a C literal: make sure there is a decimal point or an exponent before the suffix
  if (r.find('.') == std::string::npos && r.find('e') == std::string::npos && r.find("inf") == std::string::npos)
    r.insert(r.size() - 1, ".0");
  return r;
}

std::string t(int id) { return "t" + std::to_string(id); }

}  // namespace

static int32_t emit_block(const dgc_uop *ops, int32_t n_ops, const char *kernel_name, bool seq, char *out,
                          uint64_t out_cap, uint64_t *needed) {
  if (!ops || n_ops <= 0 || !kernel_name || !needed) return DGC_ERR_INVALID;
  Emit e;
  // state cells of the sequential form, in order of first use
  std::vector<int> cells;
  auto cell_var = [&](int cell) {
    for (int c : cells)
      if (c == cell) return "s" + std::to_string(cell);
    cells.push_back(cell);
    return "s" + std::to_string(cell);
  };
  if (!seq) {
    e.s += "// generated block: one thread per (frame, element) index i of `count`\n";
    e.s += "extern \"C\" __global__ void " + std::string(kernel_name) + "(float *memory, int count) {\n";
    e.line("int i = blockIdx.x * blockDim.x + threadIdx.x;");
    e.line("if (i >= count) return;");
  } else {
    for (int k = 0; k < n_ops; ++k) {
      const int op = ops[k].op;
      if (op == DGC_OP_HISTORY_READ || op == DGC_OP_HISTORY_WRITE || op == DGC_OP_PHASOR || op == DGC_OP_LATCH ||
          op == DGC_OP_ACCUM || op == DGC_OP_NOISE) {
        if (ops[k].a < 0) return DGC_ERR_INVALID;
        cell_var(ops[k].a);
      }
    }
    e.s += "// generated sequential block: one thread per lane e of `lanes`, frames i in order, state cells in registers\n";
    e.s += "extern \"C\" __global__ void " + std::string(kernel_name) + "(float *memory, int frames, int lanes) {\n";
    e.line("int e = blockIdx.x * blockDim.x + threadIdx.x;");
    e.line("if (e >= lanes) return;");
    for (int c : cells) e.line("float s" + std::to_string(c) + " = memory[" + std::to_string(c) + " + e];");
    e.line("for (int i = 0; i < frames; ++i) {");
  }
  for (int k = 0; k < n_ops; ++k) {
    const dgc_uop &u = ops[k];
    auto ok = [&](int id) { return id >= 0 && id < k; };
    auto need = [&](int cnt) {
      if (cnt >= 1 && !ok(u.a)) return false;
      if (cnt >= 2 && !ok(u.b)) return false;
      if (cnt >= 3 && !ok(u.c)) return false;
      return true;
    };
    const std::string A = t(u.a), B = t(u.b), Cc = t(u.c), R = "float " + t(k) + " = ";
    const bool b_const = ok(u.b) && ops[u.b].op == DGC_OP_CONST;
    const bool a_const = ok(u.a) && ops[u.a].op == DGC_OP_CONST;
    const float bv = b_const ? ops[u.b].imm : 0.0f;
    switch (u.op) {
      case DGC_OP_CONST: e.line(R + fl(u.imm) + ";"); break;
      case DGC_OP_LOAD: e.line(R + "memory[" + std::to_string(u.a) + " + i];"); break;           // per-frame cell
      case DGC_OP_LOAD_SCALAR: e.line(R + "memory[" + std::to_string(u.a) + "];"); break;         // frame-invariant cell
      case DGC_OP_FRAME_INDEX: e.line(R + "(float)i;"); break;
#define BIN(OPC, EXPR) case OPC: if (!need(2)) return DGC_ERR_INVALID; e.line(R + EXPR + ";"); break;
#define UN(OPC, EXPR) case OPC: if (!need(1)) return DGC_ERR_INVALID; e.line(R + EXPR + ";"); break;
      BIN(DGC_OP_ADD, A + " + " + B)
      BIN(DGC_OP_SUB, A + " - " + B)
      BIN(DGC_OP_MUL, A + " * " + B)
      case DGC_OP_DIV:
        if (!need(2)) return DGC_ERR_INVALID;
        e.line(R + (b_const ? "(" + A + " / " + fl(bv) + ")" : A + " / " + B) + ";");
        break;
      case DGC_OP_MOD:
        if (!need(2)) return DGC_ERR_INVALID;
        if (b_const && bv == 1.0f) e.line(R + "(" + A + " - floorf(" + A + "));");
        else if (b_const) e.line(R + "(" + A + " - floorf(" + A + " / " + fl(bv) + ") * " + fl(bv) + ");");
        else e.line(R + "fmodf(" + A + ", " + B + ");");
        break;
      case DGC_OP_POW:
        if (!need(2)) return DGC_ERR_INVALID;
        if (b_const && bv == 1.0f) e.line(R + A + ";");
        else if (b_const && bv == 2.0f) e.line(R + "(" + A + " * " + A + ");");
        else if (b_const && bv == 3.0f) e.line(R + "(" + A + " * " + A + " * " + A + ");");
        else if (b_const && bv == 4.0f) e.line(R + "(" + A + " * " + A + ") * (" + A + " * " + A + ");");
        else if (b_const && bv == 0.5f) e.line(R + "sqrtf(" + A + ");");
        else if (b_const && bv == 0.0f) e.line(R + "1.0f;");
        else if (!b_const && a_const) e.line(R + "expf((" + B + ") * logf(" + fl(ops[u.a].imm) + "));");
        else e.line(R + "powf(" + A + ", " + B + ");");
        break;
      BIN(DGC_OP_MIN, "fminf(" + A + ", " + B + ")")
      BIN(DGC_OP_MAX, "fmaxf(" + A + ", " + B + ")")
      UN(DGC_OP_ABS, "fabsf(" + A + ")")
      UN(DGC_OP_SIGN, "(" + A + " == 0.0f) ? 0.0f : copysignf(1.0f, " + A + ")")
      UN(DGC_OP_FLOOR, "floorf(" + A + ")")
      UN(DGC_OP_CEIL, "ceilf(" + A + ")")
      UN(DGC_OP_ROUND, "roundf(" + A + ")")
      UN(DGC_OP_SIN, "sinf(" + A + ")")
      UN(DGC_OP_COS, "cosf(" + A + ")")
      UN(DGC_OP_TAN, "tanf(" + A + ")")
      UN(DGC_OP_ATAN, "atanf(" + A + ")")
      UN(DGC_OP_TANH, "tanhf(" + A + ")")
      UN(DGC_OP_EXP, "expf(" + A + ")")
      UN(DGC_OP_LOG, "logf(" + A + ")")
      UN(DGC_OP_LOG10, "log10f(" + A + ")")
      UN(DGC_OP_SQRT, "sqrtf(" + A + ")")
      BIN(DGC_OP_AND, "(((" + A + " != 0.0f) && (" + B + " != 0.0f)) ? 1.0f : 0.0f)")
      BIN(DGC_OP_OR, "(((" + A + " != 0.0f) || (" + B + " != 0.0f)) ? 1.0f : 0.0f)")
      BIN(DGC_OP_XOR, "((((" + A + " != 0.0f) ^ (" + B + " != 0.0f))) ? 1.0f : 0.0f)")
      BIN(DGC_OP_ATAN2, "atan2f(" + A + ", " + B + ")")
      BIN(DGC_OP_GT, "(" + A + " > " + B + ") ? 1.0f : 0.0f")
      BIN(DGC_OP_GTE, "(" + A + " >= " + B + ") ? 1.0f : 0.0f")
      BIN(DGC_OP_LTE, "(" + A + " <= " + B + ") ? 1.0f : 0.0f")
      BIN(DGC_OP_LT, "(" + A + " < " + B + ") ? 1.0f : 0.0f")
      BIN(DGC_OP_EQ, "(" + A + " == " + B + ") ? 1.0f : 0.0f")
      case DGC_OP_GSWITCH:
        if (!need(3)) return DGC_ERR_INVALID;
        e.line(R + A + " > 0.0f ? " + B + " : " + Cc + ";");
        break;
      // ---- lane-indexed memory and state ops: sequential form only ----
      case DGC_OP_LOAD_LANE:
        if (!seq) return DGC_ERR_UNSUPPORTED;
        e.line(R + "memory[" + std::to_string(u.a) + " + e];");
        break;
      case DGC_OP_LOAD_FRAME_LANE:
        if (!seq) return DGC_ERR_UNSUPPORTED;
        e.line(R + "memory[" + std::to_string(u.a) + " + (size_t)i * lanes + e];");
        break;
      case DGC_OP_STORE_FRAME_LANE:
        if (!seq) return DGC_ERR_UNSUPPORTED;
        if (!ok(u.b)) return DGC_ERR_INVALID;
        e.line("memory[" + std::to_string(u.a) + " + (size_t)i * lanes + e] = " + B + ";");
        e.line(R + B + ";");
        break;
      case DGC_OP_HISTORY_READ:   // Sources/DGen/Emit+State.swift:150-224: the cell's current content
        if (!seq) return DGC_ERR_UNSUPPORTED;
        e.line(R + cell_var(u.a) + ";");
        break;
      case DGC_OP_HISTORY_WRITE:  // pass-through store: later reads (this frame or the next) see the new value
        if (!seq) return DGC_ERR_UNSUPPORTED;
        if (!ok(u.b)) return DGC_ERR_INVALID;
        e.line(cell_var(u.a) + " = " + B + ";");
        e.line(R + B + ";");
        break;
      case DGC_OP_PHASOR: {       // Sources/DGen/Definitions.swift:96-102, Emit+State.swift:322-369; imm = sample rate
        if (!seq) return DGC_ERR_UNSUPPORTED;
        if (!ok(u.b) || !ok(u.c)) return DGC_ERR_INVALID;
        const std::string S = cell_var(u.a), N = "n" + std::to_string(k);
        e.line(R + S + ";");                                       // the output is the phase BEFORE the update
        e.line("float " + N + " = " + S + " + " + B + " / " + fl(u.imm) + ";");
        e.line(N + " = " + N + " - floorf(" + N + ");");
        e.line("if (" + N + " >= 1.0f) " + N + " -= 1.0f;");
        e.line(S + " = " + Cc + " > 0.0f ? 0.0f : " + N + ";");
        break;
      }
      case DGC_OP_ACCUM: {        // Sources/DGen/Definitions.swift:215-246: cell a, increment t_b, reset t_c, range [0, imm)
        if (!seq) return DGC_ERR_UNSUPPORTED;
        if (!ok(u.b) || !ok(u.c)) return DGC_ERR_INVALID;
        const std::string S = cell_var(u.a), N = "n" + std::to_string(k), M = fl(u.imm);
        e.line(R + S + ";");                                       // the output is the state BEFORE the update
        e.line("float " + N + " = " + Cc + " > 0.0f ? 0.0f : " + S + " + " + B + ";");
        e.line(N + " = " + N + " - floorf(" + N + " / " + M + ") * " + M + ";");
        e.line("if (" + N + " >= " + M + ") " + N + " -= " + M + ";");
        e.line(S + " = " + Cc + " > 0.0f ? 0.0f : " + N + ";");
        break;
      }
      case DGC_OP_NOISE: {        // Sources/DGen/Renderer/CRenderer.swift:660-695: xorshift32, state bits in the cell
        if (!seq) return DGC_ERR_UNSUPPORTED;
        const std::string S = cell_var(u.a), X = "x" + std::to_string(k);
        e.line("unsigned " + X + " = __float_as_uint(" + S + ");");
        e.line("if (" + X + " == 0u) " + X + " = 1u;");
        e.line(X + " ^= " + X + " << 13; " + X + " ^= " + X + " >> 17; " + X + " ^= " + X + " << 5;");
        e.line(S + " = __uint_as_float(" + X + ");");
        e.line(R + "(float)" + X + " / 4294967296.0f;");
        break;
      }
      case DGC_OP_LATCH:          // Sources/DGen/Definitions.swift:104-113: cell a, value t_b, cond t_c
        if (!seq) return DGC_ERR_UNSUPPORTED;
        if (!ok(u.b) || !ok(u.c)) return DGC_ERR_INVALID;
        e.line("if (" + Cc + " > 0.0f) " + cell_var(u.a) + " = " + B + ";");
        e.line(R + cell_var(u.a) + ";");
        break;
      case DGC_OP_STORE:   // memory[a + i] = t_b ; the op's own value is the stored value
        if (!ok(u.b)) return DGC_ERR_INVALID;
        e.line("memory[" + std::to_string(u.a) + " + i] = " + B + ";");
        e.line(R + B + ";");
        break;
      case DGC_OP_OUTPUT:  // the `output` store: non-finite -> 0 (toolchain/include/dgen_runtime.h:72-74)
        if (!ok(u.b)) return DGC_ERR_INVALID;
        e.line(R + "((__float_as_uint(" + B + ") & 0x7f800000u) == 0x7f800000u) ? 0.0f : " + B + ";");
        e.line("memory[" + std::to_string(u.a) + " + i] = " + t(k) + ";");
        break;
#undef BIN
#undef UN
      default: return DGC_ERR_UNSUPPORTED;
    }
  }
  if (seq) {
    e.line("}");
    for (int c : cells) e.line("memory[" + std::to_string(c) + " + e] = s" + std::to_string(c) + ";");
  }
  e.s += "}\n";
  *needed = e.s.size() + 1;
  if (out && out_cap >= *needed) memcpy(out, e.s.c_str(), *needed);
  else if (out && out_cap > 0) out[0] = 0;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_block_emit(const dgc_uop *ops, int32_t n_ops, const char *kernel_name, char *out,
                                  uint64_t out_cap, uint64_t *needed) {
  return emit_block(ops, n_ops, kernel_name, false, out, out_cap, needed);
}

DGC_EXPORT int32_t dgc_block_emit_sequential(const dgc_uop *ops, int32_t n_ops, const char *kernel_name, char *out,
                                             uint64_t out_cap, uint64_t *needed) {
  return emit_block(ops, n_ops, kernel_name, true, out, out_cap, needed);
}

static int32_t compile_block(dgc_ctx *ctx, const dgc_uop *ops, int32_t n_ops, const char *kernel_name, bool seq,
                             dgc_module **out) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, ops && n_ops > 0 && kernel_name && out, "null argument");
  uint64_t need = 0;
  int32_t rc = emit_block(ops, n_ops, kernel_name, seq, nullptr, 0, &need);
  if (rc == DGC_ERR_UNSUPPORTED)
    return dgc_fail(ctx, rc, "block compile: an op of the list is not available in this block form");
  if (rc != DGC_OK) return dgc_fail(ctx, rc, "block compile: malformed op list (operand ids must precede their use)");
  std::string src(need, '\0');
  rc = emit_block(ops, n_ops, kernel_name, seq, &src[0], need, &need);
  if (rc != DGC_OK) return dgc_fail(ctx, rc, "block compile: emit failed");
  return dgc_module_compile(ctx, src.c_str(), kernel_name, out);
}

DGC_EXPORT int32_t dgc_block_compile(dgc_ctx *ctx, const dgc_uop *ops, int32_t n_ops, const char *kernel_name,
                                     dgc_module **out) {
  return compile_block(ctx, ops, n_ops, kernel_name, false, out);
}

DGC_EXPORT int32_t dgc_block_compile_sequential(dgc_ctx *ctx, const dgc_uop *ops, int32_t n_ops,
                                                const char *kernel_name, dgc_module **out) {
  return compile_block(ctx, ops, n_ops, kernel_name, true, out);
}
