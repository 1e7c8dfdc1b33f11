// Emitter for the elementwise blocks that no recognised primitive covers: a block is a short SSA program
// over arena cells, one thread per (frame, element) index, rendered to CUDA C with the SAME scalar
// expressions the reference's C renderer writes for each op (Sources/DGen/Renderer/CRenderer.swift:484-1040,
// scalar branch of every case; the frame loop `for (int i = 0; i < frameCount; i++)` becomes the thread
// index), then compiled for sm_100a through dgc_module_compile.  The Swift-side renderer that walks the
// reference's UOps would produce exactly this op list; it is host code of the reference and not part of
// this library.
#include <cstdio>
#include <string>

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

DGC_EXPORT int32_t dgc_block_emit(const dgc_uop *ops, int32_t n_ops, const char *kernel_name, char *out,
                                  uint64_t out_cap, uint64_t *needed) {
  if (!ops || n_ops <= 0 || !kernel_name || !needed) return DGC_ERR_INVALID;
  Emit e;
  e.s += "// generated block: one thread per (frame, element) index i of `count`\n";
  e.s += "extern \"C\" __global__ void " + std::string(kernel_name) + "(float *memory, int count) {\n";
  e.line("int i = blockIdx.x * blockDim.x + threadIdx.x;");
  e.line("if (i >= count) return;");
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
  e.s += "}\n";
  *needed = e.s.size() + 1;
  if (out && out_cap >= *needed) memcpy(out, e.s.c_str(), *needed);
  else if (out && out_cap > 0) out[0] = 0;
  return DGC_OK;
}

DGC_EXPORT int32_t dgc_block_compile(dgc_ctx *ctx, const dgc_uop *ops, int32_t n_ops, const char *kernel_name,
                                     dgc_module **out) {
  if (!ctx) return DGC_ERR_INVALID;
  DGC_REQUIRE(ctx, ops && n_ops > 0 && kernel_name && out, "null argument");
  uint64_t need = 0;
  int32_t rc = dgc_block_emit(ops, n_ops, kernel_name, nullptr, 0, &need);
  if (rc != DGC_OK) return dgc_fail(ctx, rc, "dgc_block_compile: malformed op list (operand ids must precede their use)");
  std::string src(need, '\0');
  rc = dgc_block_emit(ops, n_ops, kernel_name, &src[0], need, &need);
  if (rc != DGC_OK) return dgc_fail(ctx, rc, "dgc_block_compile: emit failed");
  return dgc_module_compile(ctx, src.c_str(), kernel_name, out);
}
