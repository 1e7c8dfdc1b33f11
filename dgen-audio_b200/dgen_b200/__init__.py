"""Host-side binding of libdgen_cuda.so (ctypes) for tests, the benchmark and Python callers.

The product is the shared library behind include/dgen_cuda.h; this module only loads it, declares
the C signatures and offers thin helpers that pass `torch` CUDA tensors as raw device pointers.
There is no CPU fallback: importing works anywhere, but every compute entry point needs the
library and a CUDA device, and raises `DgenCudaError` otherwise.
"""
import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(PKG_DIR, "libdgen_cuda.so")

DGC_OK = 0
PHASE_DETERMINISTIC, PHASE_SEQUENTIAL, PHASE_SCAN, PHASE_FUNDAMENTAL = 0, 1, 2, 3
MSS_MAX_SCALES = 8


class DgenCudaError(RuntimeError):
    pass


class HarmonicParams(C.Structure):
    _fields_ = [("B", C.c_int32), ("T", C.c_int32), ("K", C.c_int32), ("F", C.c_int32),
                ("sample_rate", C.c_float), ("harmonic_scale", C.c_float),
                ("phase_mode", C.c_int32), ("accumulate", C.c_int32)]


class FirParams(C.Structure):
    _fields_ = [("B", C.c_int32), ("T", C.c_int32), ("F", C.c_int32), ("taps", C.c_int32),
                ("scale", C.c_float), ("accumulate", C.c_int32)]


class MssParams(C.Structure):
    _fields_ = [("B", C.c_int32), ("T", C.c_int32), ("nscales", C.c_int32),
                ("sizes", C.c_int32 * MSS_MAX_SCALES), ("hop_div", C.c_int32),
                ("w_lin", C.c_float), ("w_log", C.c_float)]


class BiquadParams(C.Structure):
    _fields_ = [("B", C.c_int32), ("T", C.c_int32), ("L", C.c_int32), ("gain", C.c_float), ("mode", C.c_float)]


class CompressorParams(C.Structure):
    _fields_ = [("B", C.c_int32), ("T", C.c_int64), ("ratio", C.c_float), ("threshold", C.c_float),
                ("knee", C.c_float), ("attack", C.c_float), ("release", C.c_float), ("sample_rate", C.c_float)]


class Uop(C.Structure):
    """One op of a generated block (dgc_uop)."""
    _fields_ = [("op", C.c_int32), ("a", C.c_int32), ("b", C.c_int32), ("c", C.c_int32), ("imm", C.c_float)]


# op codes of include/dgen_cuda.h
OP = dict(CONST=0, LOAD=1, LOAD_SCALAR=2, FRAME_INDEX=3,
          ADD=10, SUB=11, MUL=12, DIV=13, MOD=14, POW=15, MIN=16, MAX=17, ATAN2=18, AND=19, OR=20, XOR=21, GT=22,
          GTE=23, LTE=24, LT=25, EQ=26,
          ABS=40, SIGN=41, FLOOR=42, CEIL=43, ROUND=44, SIN=45, COS=46, TAN=47, ATAN=48, TANH=49, EXP=50, LOG=51,
          LOG10=52, SQRT=53, GSWITCH=60, STORE=70, OUTPUT=71,
          LOAD_LANE=80, LOAD_FRAME_LANE=81, STORE_FRAME_LANE=82, HISTORY_READ=83, HISTORY_WRITE=84, PHASOR=85,
          LATCH=86, ACCUM=87, NOISE=88)


def _uops(ops):
    """ops: list of (name, a, b, c, imm) tuples (missing fields 0) -> ctypes array."""
    arr = (Uop * len(ops))()
    for k, o in enumerate(ops):
        o = tuple(o) + (0,) * (5 - len(o))
        arr[k] = Uop(OP[o[0]] if isinstance(o[0], str) else int(o[0]), int(o[1]), int(o[2]), int(o[3]), float(o[4]))
    return arr


def block_source(ops, name="dgen_block", sequential=False):
    """CUDA C source the library emits for an op list (no GPU needed).  sequential=True: the form for blocks
    with state cells, one thread per lane with the frame loop inside."""
    arr = _uops(ops)
    need = C.c_uint64(0)
    lib = load()
    emit = lib.dgc_block_emit_sequential if sequential else lib.dgc_block_emit
    rc = emit(arr, len(ops), name.encode(), None, 0, C.byref(need))
    if rc != DGC_OK:
        raise DgenCudaError("dgc_block_emit failed: %d" % rc)
    buf = C.create_string_buffer(need.value)
    rc = emit(arr, len(ops), name.encode(), buf, need.value, C.byref(need))
    if rc != DGC_OK:
        raise DgenCudaError("dgc_block_emit failed: %d" % rc)
    return buf.value.decode()


class HnStep(C.Structure):
    _fields_ = [("harm", HarmonicParams), ("fir", FirParams), ("mss", MssParams), ("nbands", C.c_int32),
                ("noise_seed", C.c_uint32), ("noise_mode", C.c_int32), ("noise_sigma", C.c_float),
                ("target_dev", C.c_void_p)]


NOISE_STREAM, NOISE_GAUSSIAN = 0, 1


_vp, _i32, _i64, _u64, _u32, _f = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_uint32, C.c_float

PLAN_NONE = 0xffffffffffffffff
(PLAN_FORK, PLAN_JOIN, PLAN_OSC_BANK_CONST, PLAN_HARMONIC_RENDER, PLAN_BANDS_TO_TAPS, PLAN_FIR_NOISE, PLAN_ADD, PLAN_COPY,
 PLAN_ONEPOLE, PLAN_BIQUAD_FWD, PLAN_BIQUAD_MSE_BWD, PLAN_STFT_MAG, PLAN_PARTCONV, PLAN_PARTCONV_BWD, PLAN_MSS_LOSS_FWD,
 PLAN_MSS_LOSS_BWD, PLAN_LINEAR_FWD, PLAN_LINEAR_BWD, PLAN_HEADS_FWD, PLAN_HEADS_BWD, PLAN_HARMONIC_BWD, PLAN_FIR_BWD,
 PLAN_ALLREDUCE, PLAN_ADAM, PLAN_SANITIZE, PLAN_BLOCK) = range(26)


class PlanStep(C.Structure):
    _fields_ = [("op", C.c_int32), ("stream", C.c_int32), ("a", C.c_uint64 * 10), ("i", C.c_int32 * 16),
                ("f", C.c_float * 4)]


def plan_step(op, a=(), i=(), f=(), stream=0):
    """One dgc_plan_step: arena offsets a (None = absent), integers i, floats f."""
    s = PlanStep()
    s.op, s.stream = op, stream
    for k in range(10):
        s.a[k] = PLAN_NONE
    for k, v in enumerate(a):
        s.a[k] = PLAN_NONE if v is None else int(v)
    for k, v in enumerate(i):
        s.i[k] = int(v)
    for k, v in enumerate(f):
        s.f[k] = float(v)
    return s


class Plan(C.Structure):
    _fields_ = [("steps", C.POINTER(PlanStep)), ("n_steps", C.c_int32), ("modules", C.POINTER(C.c_void_p)),
                ("kernels", C.POINTER(C.c_char_p)), ("n_kernels", C.c_int32)]


class HnTrainConfig(C.Structure):
    _fields_ = [("B", C.c_int32), ("T", C.c_int32), ("K", C.c_int32), ("F", C.c_int32), ("sample_rate", C.c_float),
                ("nbands", C.c_int32), ("taps", C.c_int32), ("in_features", C.c_int32), ("hidden", C.c_int32),
                ("n_trunk", C.c_int32), ("ir_len", C.c_int32), ("conv_n", C.c_int32), ("conv_hop", C.c_int32),
                ("mss", MssParams), ("phase_mode", C.c_int32), ("global_voices", C.c_int32), ("lr", C.c_float),
                ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float)]


class HnTrainLayout(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("total_floats", "n_params", "params", "grads", "adam_m", "adam_v", "adam_t",
                                          "adam_corr", "x", "f0", "uv", "gain", "noise_gain", "noise", "w_fs", "target",
                                          "loss", "audio")] + [("n_steps", C.c_int32), ("n_forward_backward", C.c_int32)]

# name -> (restype, argtypes); one line per declaration of include/dgen_cuda.h
SIGNATURES = {
    "dgc_abi_version": (_i32, []),
    "dgc_ctx_create": (_i32, [_i32, C.POINTER(_vp)]),
    "dgc_ctx_destroy": (_i32, [_vp]),
    "dgc_last_error": (C.c_char_p, [_vp]),
    "dgc_ctx_set_stream": (_i32, [_vp, _vp, _i32]),
    "dgc_selftest_expired_wait": (_i32, [_vp, _u32]),
    "dgc_selftest_busy": (_i32, [_vp, _u32]),
    "dgc_sync": (_i32, [_vp, _u32]),
    "dgc_profile_begin": (_i32, [_vp]),
    "dgc_profile_end": (_i32, [_vp, C.POINTER(_f)]),
    "dgc_launch_count": (_i64, [_vp]),
    "dgc_arena_create": (_i32, [_vp, _u64, C.POINTER(_vp)]),
    "dgc_arena_wrap": (_i32, [_vp, _vp, _u64, C.POINTER(_vp)]),
    "dgc_plan_run": (_i32, [_vp, _vp, C.POINTER(Plan), _i32, _i32]),
    "dgc_hn_train_plan": (_i32, [C.POINTER(HnTrainConfig), C.POINTER(HnTrainLayout), C.POINTER(PlanStep), _i32]),
    "dgc_arena_destroy": (_i32, [_vp]),
    "dgc_arena_ptr": (_vp, [_vp]),
    "dgc_arena_size": (_u64, [_vp]),
    "dgc_arena_zero": (_i32, [_vp]),
    "dgc_arena_upload": (_i32, [_vp, _u64, _vp, _u64]),
    "dgc_arena_download": (_i32, [_vp, _u64, _vp, _u64]),
    "dgc_clock_accum": (_i32, [_vp, _f, _f, _f, _f, _i32, _vp]),
    "dgc_playhead": (_i32, [_vp, _i32, _i32, C.POINTER(_vp)]),
    "dgc_osc_bank_const": (_i32, [_vp, _vp, _vp, _i32, _i32, _f, _i32, _vp]),
    "dgc_harmonic_scratch_floats": (_u64, [C.POINTER(HarmonicParams)]),
    "dgc_harmonic_render": (_i32, [_vp, C.POINTER(HarmonicParams), _vp, _vp, _vp, _vp, _vp, _vp]),
    "dgc_fir_noise": (_i32, [_vp, C.POINTER(FirParams), _vp, _vp, _vp, _vp]),
    "dgc_noise_fill": (_i32, [_vp, _u32, _i32, _i32, _i32, _f, _vp]),
    "dgc_bands_to_taps": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "dgc_onepole_fwd": (_i32, [_vp, _vp, _i32, _i32, _f, _vp]),
    "dgc_onepole_fwd_state": (_i32, [_vp, _vp, _i32, _i32, _f, _vp, _vp]),
    "dgc_biquad_fwd_state": (_i32, [_vp, C.POINTER(BiquadParams), _vp, _vp, _vp, _vp, _vp, _vp]),
    "dgc_onepole_fwd_static": (_i32, [_vp, _vp, _i32, _i32, _f, _vp, C.c_char_p, _u32]),
    "dgc_biquad_scratch_floats": (_u64, [C.POINTER(BiquadParams), _i32]),
    "dgc_biquad_fwd": (_i32, [_vp, C.POINTER(BiquadParams), _vp, _vp, _vp, _vp, _vp]),
    "dgc_biquad_mse_bwd": (_i32, [_vp, C.POINTER(BiquadParams), _vp, _vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _vp]),
    "dgc_stft_mag": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "dgc_partconv_scratch_floats": (_u64, [_i32, _i32, _i32, _i32, _i32]),
    "dgc_partconv": (_i32, [_vp, _vp, _i32, _i32, _vp, _i32, _i32, _i32, _f, _vp, _i32, _vp]),
    "dgc_mss_partial_floats": (_u64, [C.POINTER(MssParams)]),
    "dgc_mss_loss_fwd": (_i32, [_vp, C.POINTER(MssParams), _vp, _vp, _vp, _vp]),
    "dgc_mss_loss_bwd": (_i32, [_vp, C.POINTER(MssParams), _vp, _vp, _f, _vp]),
    "dgc_harmonic_bwd_scratch_floats": (_u64, [C.POINTER(HarmonicParams)]),
    "dgc_harmonic_render_bwd": (_i32, [_vp, C.POINTER(HarmonicParams), _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dgc_fir_noise_bwd": (_i32, [_vp, C.POINTER(FirParams), _vp, _vp, _vp, _vp]),
    "dgc_hn_heads_fwd": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "dgc_hn_heads_bwd": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "dgc_partconv_bwd_scratch_floats": (_u64, [_i32, _i32, _i32, _i32, _i32]),
    "dgc_partconv_bwd": (_i32, [_vp, _vp, _i32, _i32, _vp, _i32, _i32, _i32, _f, _vp, _vp, _i32, _vp, _vp]),
    "dgc_linear_fwd": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "dgc_linear_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp]),
    "dgc_gemm_path_counts": (_i32, [_vp, C.POINTER(C.c_int64)]),
    "dgc_adam_step": (_i32, [_vp, _vp, _vp, _vp, _vp, _u64, _i32, _f, _f, _f, _f]),
    "dgc_sanitize": (_i32, [_vp, _vp, _u64, _vp]),
    "dgc_reduce_frames": (_i32, [_vp, _vp, _i64, _i64, _f, _i32, _vp]),
    "dgc_onepole_bwd": (_i32, [_vp, _vp, _vp, _i32, _i32, _f, _vp, _vp]),
    "dgc_biquad_bwd": (_i32, [_vp, C.POINTER(BiquadParams)] + [_vp] * 9),
    "dgc_adam_step_counted": (_i32, [_vp, _vp, _vp, _vp, _vp, _u64, _vp, _vp, _f, _f, _f, _f]),
    "dgc_graph_begin": (_i32, [_vp]),
    "dgc_graph_end": (_i32, [_vp, C.POINTER(_vp)]),
    "dgc_graph_nodes": (_u64, [_vp]),
    "dgc_graph_launch": (_i32, [_vp, _vp]),
    "dgc_graph_destroy": (_i32, [_vp]),
    "dgc_stft_scratch_floats": (_u64, [_i32, _i32, _i32, _i32, _i32]),
    "dgc_stft_fwd": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "dgc_istft_ola": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _f, _vp, _i32, _vp]),
    "dgc_phase_vocoder_scratch_floats": (_u64, [_i32, _i64, _i32]),
    "dgc_phase_vocoder": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i64, _i32, _i32, _vp, _vp, _vp, _vp]),
    "dgc_delay_line": (_i32, [_vp, _vp, _vp, _i32, _i64, _i32, _i32, _vp, _vp, _vp]),
    "dgc_spectrum_delay": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _vp, _vp, _vp]),
    "dgc_latch_scratch_floats": (_u64, [_i64, _i32]),
    "dgc_latch": (_i32, [_vp, _vp, _vp, _i32, _i64, _i32, _vp, _vp, _vp]),
    "dgc_compressor": (_i32, [_vp, C.POINTER(CompressorParams), _vp, _vp, _vp, _vp]),
    "dgc_ctx_prepare_tables": (_i32, [_vp, _i32, _i32]),
    "dgc_module_load": (_i32, [_vp, _vp, _u64, C.POINTER(_vp)]),
    "dgc_module_compile": (_i32, [_vp, C.c_char_p, C.c_char_p, C.POINTER(_vp)]),
    "dgc_module_unload": (_i32, [_vp]),
    "dgc_launch": (_i32, [_vp, C.c_char_p, C.POINTER(_u32), C.POINTER(_u32), _u32, C.POINTER(_vp)]),
    "dgc_block_emit": (_i32, [C.POINTER(Uop), _i32, C.c_char_p, C.c_char_p, _u64, C.POINTER(_u64)]),
    "dgc_block_compile": (_i32, [_vp, C.POINTER(Uop), _i32, C.c_char_p, C.POINTER(_vp)]),
    "dgc_block_emit_sequential": (_i32, [C.POINTER(Uop), _i32, C.c_char_p, C.c_char_p, _u64, C.POINTER(_u64)]),
    "dgc_block_compile_sequential": (_i32, [_vp, C.POINTER(Uop), _i32, C.c_char_p, C.POINTER(_vp)]),
    "dgc_comm_unique_id": (_i32, [C.c_char_p]),
    "dgc_comm_init": (_i32, [_vp, _i32, _i32, C.c_char_p]),
    "dgc_allreduce_sum": (_i32, [_vp, _vp, _u64]),
    "dgc_comm_destroy": (_i32, [_vp]),
    "dgc_harmonic_render_bwd_prepared": (_i32, [_vp, C.POINTER(HarmonicParams), _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dgc_harmonic_f0_bwd_scratch_floats": (_u64, [C.POINTER(HarmonicParams)]),
    "dgc_harmonic_f0_bwd": (_i32, [_vp, C.POINTER(HarmonicParams), _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dgc_temporal_grad_scan": (_i32, [_vp, _vp, _vp, _i32, _i32, _f, _vp]),
    "dgc_hn_forward_loss_work_floats": (_u64, [C.POINTER(HnStep)]),
    "dgc_hn_forward_loss": (_i32, [_vp, C.POINTER(HnStep)] + [_vp] * 9 + [_vp, _vp, _vp]),
    "dgc_hn_forward_loss_host": (_i32, [_vp, C.POINTER(HnStep)] + [_vp] * 9 + [C.POINTER(C.c_double), _vp]),
    "dgc_hn_forward_loss_host_submit": (_i32, [_vp, C.POINTER(HnStep)] + [_vp] * 9 + [_i32, _vp, _vp]),
    "dgc_hn_forward_loss_host_wait": (_i32, [_vp, _i32]),
}

_lib = None


def comm_unique_id():
    """128 bytes that rank 0 creates and every rank passes to Context.comm_init."""
    buf = C.create_string_buffer(128)
    rc = load().dgc_comm_unique_id(buf)
    if rc != DGC_OK:
        raise DgenCudaError("dgc_comm_unique_id failed: %d (NCCL not found?)" % rc)
    return buf.raw


class Module:
    """A loaded set of generated kernels (dgc_module)."""

    def __init__(self, ctx, handle):
        self.ctx, self.h = ctx, handle

    def launch(self, name, grid, block, args, smem=0):
        """args: ctypes scalars (c_int, c_float, ...) or torch CUDA tensors (passed as device pointers)."""
        def dim3(v):
            v = tuple(v) if isinstance(v, (tuple, list)) else (v,)
            return (_u32 * 3)(*(v + (1, 1, 1))[:3])
        keep = [a if isinstance(a, C._SimpleCData) else _vp(a.data_ptr()) for a in args]
        argv = (_vp * max(1, len(keep)))(*[C.cast(C.byref(k), _vp) for k in keep])
        self.ctx.check(self.ctx.lib.dgc_launch(self.h, name.encode(), dim3(grid), dim3(block), smem, argv))

    def close(self):
        if self.h:
            self.ctx.lib.dgc_module_unload(self.h)
            self.h = None


def load():
    """Load libdgen_cuda.so (built in-tree by dgen-audio_b200/build.py).  Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise DgenCudaError("libdgen_cuda.so not found at %s: run `python dgen-audio_b200/build.py` "
                            "(there is no CPU fallback)" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def mss_params(B, T, sizes=(2048, 1024, 512, 256, 128, 64), hop_div=4, w_lin=1.0, w_log=1.0):
    p = MssParams()
    p.B, p.T, p.nscales, p.hop_div, p.w_lin, p.w_log = B, T, len(sizes), hop_div, w_lin, w_log
    for i, s in enumerate(sizes):
        p.sizes[i] = s
    return p


def _ptr(t):
    """Device pointer of a contiguous float32 CUDA tensor (or None)."""
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "expected a contiguous CUDA tensor"
    return t.data_ptr()


class StepGraph:
    """A recorded step (dgc_graph): launch() replays it on the context's stream."""

    def __init__(self, ctx, handle):
        self.ctx, self.h = ctx, handle

    @property
    def nodes(self):
        return int(self.ctx.lib.dgc_graph_nodes(self.h))

    def launch(self):
        self.ctx.check(self.ctx.lib.dgc_graph_launch(self.ctx.h, self.h))

    def close(self):
        if self.h:
            self.ctx.lib.dgc_graph_destroy(self.h)
            self.h = None


class _Recording:
    def __init__(self, ctx):
        self.ctx, self.graph = ctx, None

    def __enter__(self):
        self.ctx.check(self.ctx.lib.dgc_graph_begin(self.ctx.h))
        return self

    def __exit__(self, et, ev, tb):
        out = _vp()
        rc = self.ctx.lib.dgc_graph_end(self.ctx.h, C.byref(out))
        if et is None:
            self.ctx.check(rc)
            self.graph = StepGraph(self.ctx, out)
        elif rc == 0 and out:
            self.ctx.lib.dgc_graph_destroy(out)
        return False


class Context:
    """One dgc_ctx on one GPU.  Methods take torch CUDA tensors and enqueue on torch's current stream."""

    def __init__(self, device=0, use_torch_stream=True):
        import torch
        if not torch.cuda.is_available():
            raise DgenCudaError("no CUDA device: libdgen_cuda has no CPU path")
        self.lib = load()
        self.torch = torch
        self.device = device
        torch.cuda.set_device(device)
        h = _vp()
        rc = self.lib.dgc_ctx_create(device, C.byref(h))
        if rc != DGC_OK:
            raise DgenCudaError("dgc_ctx_create failed: %d" % rc)
        self.h = h
        if use_torch_stream:
            self.check(self.lib.dgc_ctx_set_stream(self.h, torch.cuda.current_stream(device).cuda_stream, 1))

    def on_stream(self, stream):
        """Context manager: library calls inside run on `stream` (a torch.cuda.Stream); the binding to torch's
        current stream is restored on exit."""
        import contextlib

        @contextlib.contextmanager
        def scope():
            self.check(self.lib.dgc_ctx_set_stream(self.h, stream.cuda_stream, 1))
            try:
                yield
            finally:
                self.check(self.lib.dgc_ctx_set_stream(self.h, self.torch.cuda.current_stream(self.device).cuda_stream, 1))
        return scope()

    def close(self):
        if getattr(self, "h", None):
            self.lib.dgc_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, rc):
        if rc != DGC_OK:
            raise DgenCudaError("libdgen_cuda error %d: %s" % (rc, self.lib.dgc_last_error(self.h).decode()))

    def sync(self, timeout_ms=0):
        self.check(self.lib.dgc_sync(self.h, timeout_ms))

    def launch_count(self):
        return self.lib.dgc_launch_count(self.h)

    def gemm_path_counts(self):
        """(simt, tcgen05 generic, tcgen05 pipeline, tcgen05 pipeline with wide tiles) products issued so far."""
        out = (C.c_int64 * 4)()
        self.check(self.lib.dgc_gemm_path_counts(self.h, out))
        return tuple(out)

    def _empty(self, *shape, dtype=None):
        return self.torch.empty(*shape, dtype=dtype or self.torch.float32, device="cuda:%d" % self.device)

    # ---- clocks -----------------------------------------------------------------------------
    def clock_accum(self, incr, mn, mx, T, state0=0.0):
        out = self._empty(T)
        self.check(self.lib.dgc_clock_accum(self.h, incr, mn, mx, state0, T, _ptr(out)))
        return out

    def playhead(self, F, T):
        """Copy of the context's cached control clock for (F, T) in a tensor the caller owns."""
        p = _vp()
        self.check(self.lib.dgc_playhead(self.h, F, T, C.byref(p)))
        out = self._empty(T)
        self.torch.cuda.synchronize()
        rc = _cudart().cudaMemcpy(C.c_void_p(out.data_ptr()), p, C.c_size_t(4 * T), 3)  # device to device
        if rc != 0:
            raise DgenCudaError("cudaMemcpy of the playhead failed: %d" % rc)
        return out

    # ---- oscillator bank ----------------------------------------------------------------------
    def osc_bank_const(self, freq, amp, T, sr, phase_mode=PHASE_DETERMINISTIC):
        out = self._empty(T)
        self.check(self.lib.dgc_osc_bank_const(self.h, _ptr(freq), _ptr(amp), freq.numel(), T, sr, phase_mode,
                                               _ptr(out)))
        return out

    def harmonic_render(self, f0, uv, amps, gain, T, sr, phase_mode=PHASE_SCAN, scale=1.0, out=None,
                        accumulate=False, scratch=None):
        F, B = f0.shape
        K = amps.shape[2]
        p = HarmonicParams(B, T, K, F, sr, scale, phase_mode, int(accumulate))
        if out is None:
            out = self._empty(B, T)
        self.check(self.lib.dgc_harmonic_render(self.h, C.byref(p), _ptr(f0), _ptr(uv), _ptr(amps), _ptr(gain),
                                                _ptr(scratch), _ptr(out)))
        return out

    def harmonic_scratch_floats(self, B, T, K, F):
        p = HarmonicParams(B, T, K, F, 1.0, 1.0, PHASE_SCAN, 0)
        return self.lib.dgc_harmonic_scratch_floats(C.byref(p))

    def fir_noise(self, noise, taps, noise_gain, scale=0.12, out=None, accumulate=False):
        F, B, NT = taps.shape
        T = noise.shape[1]
        p = FirParams(B, T, F, NT, scale, int(accumulate))
        if out is None:
            out = self._empty(B, T)
        self.check(self.lib.dgc_fir_noise(self.h, C.byref(p), _ptr(noise), _ptr(taps), _ptr(noise_gain), _ptr(out)))
        return out

    def noise_fill(self, seed, B, T, mode=NOISE_STREAM, sigma=1.0, out=None):
        """Signal.noise() generated on the device: the reference stream (NOISE_STREAM, the same for every voice) or
        per-voice white N(0, sigma) (NOISE_GAUSSIAN)."""
        y = self._empty(B, T) if out is None else out
        self.check(self.lib.dgc_noise_fill(self.h, seed & 0xFFFFFFFF, mode, B, T, sigma, _ptr(y)))
        return y

    def bands_to_taps(self, bands, w):
        F, B, NB = bands.shape
        NT = w.shape[0]
        out = self._empty(F, B, NT)
        self.check(self.lib.dgc_bands_to_taps(self.h, _ptr(bands), _ptr(w), F * B, NB, NT, _ptr(out)))
        return out

    # ---- linear recurrences -------------------------------------------------------------------
    def onepole_fwd(self, x, a, out=None, state=None):
        """state [B] (optional): y[-1] per voice on entry, y[T-1] on return (updated in place)."""
        B, T = x.shape
        y = self._empty(B, T) if out is None else out
        if state is None:
            self.check(self.lib.dgc_onepole_fwd(self.h, _ptr(x), B, T, a, _ptr(y)))
        else:
            self.check(self.lib.dgc_onepole_fwd_state(self.h, _ptr(x), B, T, a, _ptr(state), _ptr(y)))
        return y

    def biquad_fwd(self, x, cutoff, q, gain=1.0, mode=0.0, state=None):
        """state [B][4][L] (optional): the four history cells y1, y2, x1, x2, continued from and updated in place."""
        B, T = x.shape
        L = cutoff.numel()
        p = BiquadParams(B, T, L, gain, mode)
        y = self._empty(B, T, L)
        if state is None:
            self.check(self.lib.dgc_biquad_fwd(self.h, C.byref(p), _ptr(x), _ptr(cutoff), _ptr(q), None, _ptr(y)))
        else:
            self.check(self.lib.dgc_biquad_fwd_state(self.h, C.byref(p), _ptr(x), _ptr(cutoff), _ptr(q), None,
                                                     _ptr(state), _ptr(y)))
        return y

    def biquad_mse_bwd(self, x, cutoff, q, y, target, loss_scale=1.0, gain=1.0, mode=0.0):
        B, T = x.shape
        L = cutoff.numel()
        p = BiquadParams(B, T, L, gain, mode)
        gc, gq = self._empty(L), self._empty(L)
        loss = self._empty(1, dtype=self.torch.float64)
        self.check(self.lib.dgc_biquad_mse_bwd(self.h, C.byref(p), _ptr(x), _ptr(cutoff), _ptr(q), _ptr(y),
                                               _ptr(target), loss_scale, None, _ptr(gc), _ptr(gq), _ptr(loss)))
        return gc, gq, loss

    def biquad_bwd(self, x, cutoff, q, y, gy, want_grad_x=True, gain=1.0, mode=0.0):
        """Backward for an arbitrary upstream gradient gy [B][T][L] -> (grad_cutoff [L], grad_q [L], grad_x [B][T] | None)."""
        B, T = x.shape
        L = cutoff.numel()
        p = BiquadParams(B, T, L, gain, mode)
        gc, gq = self._empty(L), self._empty(L)
        gx = self._empty(B, T) if want_grad_x else None
        self.check(self.lib.dgc_biquad_bwd(self.h, C.byref(p), _ptr(x), _ptr(cutoff), _ptr(q), _ptr(y), _ptr(gy), None,
                                           _ptr(gc), _ptr(gq), _ptr(gx) if want_grad_x else None))
        return gc, gq, gx

    def onepole_bwd(self, gy, a, y=None):
        """-> (grad_x [B][T], grad_a [B] | None): grad_a only when the forward output y is given."""
        B, T = gy.shape
        gx = self._empty(B, T)
        ga = self._empty(B) if y is not None else None
        self.check(self.lib.dgc_onepole_bwd(self.h, _ptr(y) if y is not None else None, _ptr(gy), B, T, a, _ptr(gx),
                                            _ptr(ga) if y is not None else None))
        return gx, ga

    # ---- hop-gated spectral blocks ------------------------------------------------------------
    def stft_mag(self, x, N, hop, window=None):
        V, T = x.shape
        H = (T + hop - 1) // hop
        out = self._empty(V, H, N // 2 + 1)
        self.check(self.lib.dgc_stft_mag(self.h, _ptr(x), V, T, N, hop, _ptr(window), _ptr(out)))
        return out

    def partconv(self, x, ir, N, hop, gain=1.0, out=None, accumulate=False):
        V, T = x.shape
        if out is None:
            out = self._empty(V, T)
        self.check(self.lib.dgc_partconv(self.h, _ptr(x), V, T, _ptr(ir), ir.numel(), N, hop, gain, None,
                                         int(accumulate), _ptr(out)))
        return out

    # ---- spectral loss ------------------------------------------------------------------------
    def mss_loss_fwd(self, pred, target, sizes=(2048, 1024, 512, 256, 128, 64), hop_div=4, w_lin=1.0, w_log=1.0,
                     want_partial=False):
        B, T = pred.shape
        p = mss_params(B, T, sizes, hop_div, w_lin, w_log)
        loss = self._empty(1, dtype=self.torch.float64)
        part = None
        if want_partial:
            part = self._empty(int(self.lib.dgc_mss_partial_floats(C.byref(p))))
        self.check(self.lib.dgc_mss_loss_fwd(self.h, C.byref(p), _ptr(pred), _ptr(target), _ptr(part), _ptr(loss)))
        return (loss, part) if want_partial else loss

    def mss_loss_bwd(self, pred, target, sizes=(2048, 1024, 512, 256, 128, 64), hop_div=4, w_lin=1.0, w_log=1.0,
                     upstream=1.0, out=None):
        B, T = pred.shape
        p = mss_params(B, T, sizes, hop_div, w_lin, w_log)
        grad = self._empty(B, T) if out is None else out
        self.check(self.lib.dgc_mss_loss_bwd(self.h, C.byref(p), _ptr(pred), _ptr(target), upstream, _ptr(grad)))
        return grad

    # ---- backward of the synthesis ------------------------------------------------------------
    def harmonic_render_bwd(self, f0, uv, amps, gain, g_audio, T, sr, phase_mode=PHASE_SCAN, scale=1.0):
        F, B = f0.shape
        K = amps.shape[2]
        p = HarmonicParams(B, T, K, F, sr, scale, phase_mode, 0)
        g = self._empty(F, B, K)
        self.check(self.lib.dgc_harmonic_render_bwd(self.h, C.byref(p), _ptr(f0), _ptr(uv), _ptr(amps), _ptr(gain),
                                                    _ptr(g_audio), None, _ptr(g)))
        return g

    def harmonic_f0_bwd(self, f0, uv, amps, gain, g_audio, T, sr, scale=1.0):
        """d loss / d f0 [F][B] through the phases (temporal gradient of the phasor)."""
        F, B = f0.shape
        K = amps.shape[2]
        p = HarmonicParams(B, T, K, F, sr, scale, PHASE_SCAN, 0)
        g = self._empty(F, B)
        self.check(self.lib.dgc_harmonic_f0_bwd(self.h, C.byref(p), _ptr(f0), _ptr(uv), _ptr(amps), _ptr(gain),
                                                _ptr(g_audio), None, _ptr(g)))
        return g

    def temporal_grad_scan(self, g, scale=1.0, reset=None):
        """out[e][n] = scale * sum of g[e][m] over n < m <= (first frame after n with reset > 0, or the last
        frame); 0 on a reset frame.  reset [T] or None."""
        E, T = g.shape
        out = self._empty(E, T)
        self.check(self.lib.dgc_temporal_grad_scan(self.h, _ptr(g), _ptr(reset) if reset is not None else None, E, T,
                                                   scale, _ptr(out)))
        return out

    def fir_noise_bwd(self, noise, noise_gain, g_audio, F, taps, scale=0.12):
        B, T = noise.shape
        p = FirParams(B, T, F, taps, scale, 0)
        g = self._empty(F, B, taps)
        self.check(self.lib.dgc_fir_noise_bwd(self.h, C.byref(p), _ptr(noise), _ptr(noise_gain), _ptr(g_audio),
                                              _ptr(g)))
        return g

    def heads_fwd(self, z, K):
        M, W = z.shape
        amps, bands = self._empty(M, K), self._empty(M, W - K)
        self.check(self.lib.dgc_hn_heads_fwd(self.h, _ptr(z), M, K, W - K, _ptr(amps), _ptr(bands)))
        return amps, bands

    def heads_bwd(self, z, g_amps, g_bands):
        M, W = z.shape
        K = g_amps.shape[1]
        gz = self._empty(M, W)
        self.check(self.lib.dgc_hn_heads_bwd(self.h, _ptr(z), _ptr(g_amps), _ptr(g_bands), M, K, W - K, _ptr(gz)))
        return gz

    def partconv_bwd(self, x, ir, N, hop, g_out, gain=1.0, need_gx=True, need_gir=True, gx_accumulate_into=None,
                     gir_out=None):
        """gx_accumulate_into: a [V][T] tensor that receives += A^T g_out (it may be g_out itself)."""
        V, T = x.shape
        acc = gx_accumulate_into is not None
        gx = (gx_accumulate_into if acc else self._empty(V, T)) if need_gx else None
        gir = (gir_out if gir_out is not None else self._empty(ir.numel())) if need_gir else None
        self.check(self.lib.dgc_partconv_bwd(self.h, _ptr(x), V, T, _ptr(ir), ir.numel(), N, hop, gain, _ptr(g_out),
                                             None, int(acc), _ptr(gx), _ptr(gir)))
        return gx, gir

    # ---- controller ---------------------------------------------------------------------------
    def linear_fwd(self, a, w, bias=None, act=0, want_transposed=False):
        M, K = a.shape
        N = w.shape[1]
        c = self._empty(M, N)
        ct = self._empty(N, M) if want_transposed else None
        self.check(self.lib.dgc_linear_fwd(self.h, _ptr(a), _ptr(w), _ptr(bias), M, K, N, act, _ptr(c), _ptr(ct)))
        return (c, ct) if want_transposed else c

    def linear_bwd(self, a, w, c, dc, act=0, need_da=True, need_db=True, a_t=None):
        M, K = a.shape
        N = w.shape[1]
        dz, dw = self._empty(M, N), self._empty(K, N)
        da = self._empty(M, K) if need_da else None
        db = self._empty(N) if need_db else None
        self.check(self.lib.dgc_linear_bwd(self.h, _ptr(a), _ptr(w), _ptr(c), _ptr(dc), M, K, N, act, _ptr(dz),
                                           _ptr(da), _ptr(dw), _ptr(db), _ptr(a_t)))
        return da, dw, db

    def adam_step(self, theta, grad, m, v, t, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8):
        self.check(self.lib.dgc_adam_step(self.h, _ptr(theta), _ptr(grad), _ptr(m), _ptr(v), theta.numel(), t, lr,
                                          beta1, beta2, eps))

    def adam_step_counted(self, theta, grad, m, v, t_dev, corr, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8):
        """Adam with the step index in device memory (t_dev: int32 [1], corr: float32 [2] work cell)."""
        self.check(self.lib.dgc_adam_step_counted(self.h, _ptr(theta), _ptr(grad), _ptr(m), _ptr(v), theta.numel(),
                                                  _ptr(t_dev), _ptr(corr), lr, beta1, beta2, eps))

    def record(self):
        """Context manager: library calls (and torch work on the same stream) inside are recorded, not run;
        `.graph` afterwards holds the StepGraph to replay.  The context must be on a non-default stream."""
        return _Recording(self)

    def reduce_frames(self, x, scale=1.0, out=None, accumulate=False):
        """x [T][...] -> sum over the first axis (Sources/DGen/Emit+State.swift:50-115), fixed summation order."""
        T = x.shape[0]
        E = x.numel() // T
        out = self._empty(*x.shape[1:]) if out is None else out
        self.check(self.lib.dgc_reduce_frames(self.h, _ptr(x), T, E, scale, 1 if accumulate else 0, _ptr(out)))
        return out

    def sanitize(self, x, out=None):
        """Non-finite -> 0 (toolchain/include/dgen_runtime.h:72-84); in place when out is None."""
        out = x if out is None else out
        self.check(self.lib.dgc_sanitize(self.h, _ptr(x), x.numel(), _ptr(out)))
        return out

    # ---- ring and hold ops ---------------------------------------------------------------------
    def delay_line(self, x, delay, max_delay, ring=None, head=None, per_lane=False):
        """x [T][lanes]; delay: float, or a tensor of shape [1], [T], [T][lanes] or [lanes] (Sources/DGen/Emit.swift:331-403);
        per_lane=True reads a 1-D delay as [lanes] when T == lanes makes it ambiguous.
        ring [lanes][max_delay] and head [1] are updated in place when given."""
        torch = self.torch
        T, lanes = x.shape
        if not torch.is_tensor(delay):
            delay = torch.full((1,), float(delay), dtype=torch.float32, device=x.device)
        if delay.numel() == 1:
            mode = 0
        elif delay.dim() == 2 and tuple(delay.shape) == (T, lanes):
            mode = 2
        elif delay.dim() == 1 and delay.numel() == T and not (T == lanes and per_lane):
            mode = 1
        elif delay.dim() == 1 and delay.numel() == lanes:
            mode = 3
        else:
            raise ValueError("delay must have 1, T, lanes or T*lanes elements")
        y = torch.empty_like(x)
        self.check(self.lib.dgc_delay_line(self.h, _ptr(x), _ptr(delay), mode, T, lanes, max_delay,
                                           _ptr(ring) if ring is not None else None,
                                           _ptr(head) if head is not None else None, _ptr(y)))
        return y

    def spectrum_delay(self, spec, hops, delay=None, ring=None, row=None):
        """spec [H][N]; delay None (exactly `hops` boundaries) or [H] in hops (Sources/DGen/Emit.swift:405-512)."""
        H, N = spec.shape
        out = self.torch.empty_like(spec)
        self.check(self.lib.dgc_spectrum_delay(self.h, _ptr(spec), _ptr(delay) if delay is not None else None, H, N,
                                               hops, _ptr(ring) if ring is not None else None,
                                               _ptr(row) if row is not None else None, _ptr(out)))
        return out

    def latch(self, value, cond, state=None):
        """value [T][lanes]; cond [T] or [T][lanes]; state [lanes] updated in place (Sources/DGen/Emit+State.swift:225-262)."""
        T, lanes = value.shape
        mode = 1 if cond.dim() == 1 else 2
        y = self.torch.empty_like(value)
        self.check(self.lib.dgc_latch(self.h, _ptr(value), _ptr(cond), mode, T, lanes,
                                      _ptr(state) if state is not None else None, None, _ptr(y)))
        return y

    def compressor(self, x, ratio, threshold, knee, attack, release, sample_rate, sidechain=None, state=None):
        """x [B][T] (Sources/DGen/HigherOps.swift:566-651); state [B] updated in place."""
        B, T = x.shape
        p = CompressorParams(B, T, ratio, threshold, knee, attack, release, sample_rate)
        y = self.torch.empty_like(x)
        self.check(self.lib.dgc_compressor(self.h, C.byref(p), _ptr(x), _ptr(sidechain) if sidechain is not None else None,
                                           _ptr(state) if state is not None else None, _ptr(y)))
        return y

    def stft(self, x, N, hop, window=None):
        """x [V][T] -> (re, im) [V][H][N], all bins of every hop's buffer window (Sources/DGen/HigherOps.swift:738-792,
        Sources/DGen/Emit+AcceleratedFFT.swift:16-112)."""
        V, T = x.shape
        H = (T + hop - 1) // hop
        re = self.torch.empty(V, H, N, dtype=self.torch.float32, device=x.device)
        im = self.torch.empty_like(re)
        self.check(self.lib.dgc_stft_fwd(self.h, _ptr(x), V, T, N, hop, _ptr(window) if window is not None else None,
                                         None, _ptr(re), _ptr(im)))
        return re, im

    def istft_ola(self, re, im, T, hop, window=None, gain=1.0, out=None, accumulate=False):
        """(re, im) [V][H][N] -> [V][T]: inverse FFT, window, overlap-add (Sources/DGen/Emit+FFT.swift:6-62)."""
        V, H, N = re.shape
        if H != (T + hop - 1) // hop:
            raise ValueError("spectra hold %d hops, T / hop needs %d" % (H, (T + hop - 1) // hop))
        out = self.torch.empty(V, T, dtype=self.torch.float32, device=re.device) if out is None else out
        self.check(self.lib.dgc_istft_ola(self.h, _ptr(re), _ptr(im), V, T, N, hop,
                                          _ptr(window) if window is not None else None, gain, None,
                                          1 if accumulate else 0, _ptr(out)))
        return out

    def phase_vocoder(self, re, im, ratio, hop, state=None):
        """(re, im) [V][H][N]; ratio: float, [H] or [V][H]; state [V][2N+1] updated in place
        (Sources/DGen/Emit+PhaseVocoder.swift:6-118)."""
        torch = self.torch
        V, H, N = re.shape
        if not torch.is_tensor(ratio):
            ratio = torch.full((1,), float(ratio), dtype=torch.float32, device=re.device)
        mode = 0 if ratio.numel() == 1 else (2 if ratio.dim() == 2 else 1)
        if mode == 1 and ratio.numel() != H or mode == 2 and tuple(ratio.shape) != (V, H):
            raise ValueError("ratio must have 1, H or V*H elements")
        out_re, out_im = torch.empty_like(re), torch.empty_like(im)
        self.check(self.lib.dgc_phase_vocoder(self.h, _ptr(re), _ptr(im), _ptr(ratio), mode, V, H, N, hop,
                                              _ptr(state) if state is not None else None, None, _ptr(out_re),
                                              _ptr(out_im)))
        return out_re, out_im

    # ---- generated blocks ----------------------------------------------------------------------
    def compile_module(self, cuda_source, name="dgen_block.cu"):
        """CUDA C source of generated blocks -> Module (NVRTC, sm_100a)."""
        m = _vp()
        self.check(self.lib.dgc_module_compile(self.h, cuda_source.encode(), name.encode(), C.byref(m)))
        return Module(self, m)

    def compile_block(self, ops, name="dgen_block", sequential=False):
        """Op list (see block_source) -> Module with one kernel `name(float *memory, int count)`, or
        `name(float *memory, int frames, int lanes)` for the sequential form."""
        arr = _uops(ops)
        m = _vp()
        fn = self.lib.dgc_block_compile_sequential if sequential else self.lib.dgc_block_compile
        self.check(fn(self.h, arr, len(ops), name.encode(), C.byref(m)))
        return Module(self, m)

    def load_module(self, image):
        """cubin bytes or PTX text -> Module."""
        if isinstance(image, str):
            image = image.encode() + b"\0"
        m = _vp()
        self.check(self.lib.dgc_module_load(self.h, image, len(image), C.byref(m)))
        return Module(self, m)

    # ---- gradient exchange ---------------------------------------------------------------------
    def comm_init(self, world, rank, uid):
        self.check(self.lib.dgc_comm_init(self.h, world, rank, uid))

    def allreduce_sum_(self, buf):
        self.check(self.lib.dgc_allreduce_sum(self.h, _ptr(buf), buf.numel()))
        return buf

    # ---- composite, host buffers --------------------------------------------------------------
    def hn_forward_loss(self, step, f0, uv, amps, gain, noise_gain, taps_or_bands, w, noise, target, work=None,
                        loss=None, audio=None):
        """Device-resident forward + loss (dgc_hn_forward_loss); returns (loss tensor [1] float64, work buffer)."""
        torch = self.torch
        if work is None:
            work = self._empty(int(self.lib.dgc_hn_forward_loss_work_floats(C.byref(step))))
        if loss is None:
            loss = torch.zeros(1, dtype=torch.float64, device=f0.device)
        self.check(self.lib.dgc_hn_forward_loss(self.h, C.byref(step), _ptr(f0), _ptr(uv), _ptr(amps), _ptr(gain),
                                                _ptr(noise_gain), _ptr(taps_or_bands), _ptr(w), _ptr(noise),
                                                _ptr(target), _ptr(work), _ptr(loss), _ptr(audio)))
        return loss, work

    def hn_forward_loss_host(self, step, f0, uv, amps, gain, noise_gain, taps_or_bands, w, noise, target,
                             audio_out=None):
        """All array arguments are host numpy float32 arrays or pinned CPU torch tensors."""
        def hp(a):
            if a is None:
                return None
            if hasattr(a, "data_ptr"):
                return a.data_ptr()
            return a.ctypes.data
        loss = C.c_double(0.0)
        self.check(self.lib.dgc_hn_forward_loss_host(self.h, C.byref(step), hp(f0), hp(uv), hp(amps), hp(gain),
                                                     hp(noise_gain), hp(taps_or_bands), hp(w), hp(noise),
                                                     hp(target), C.byref(loss), hp(audio_out)))
        return loss.value


    def hn_forward_loss_host_submit(self, step, f0, uv, amps, gain, noise_gain, taps_or_bands, w, noise, target, slot,
                                    audio_out=None):
        """Enqueue one host-buffer step on slot 0 or 1 and return at once; hn_forward_loss_host_wait(slot) returns its
        loss.  The arrays must be pinned and stay untouched until the wait."""
        def hp(a):
            if a is None:
                return None
            return a.data_ptr() if hasattr(a, "data_ptr") else a.ctypes.data
        if getattr(self, "_pipe_loss", None) is None:
            self._pipe_loss = self.torch.zeros(2, dtype=self.torch.float64).pin_memory()
        self.check(self.lib.dgc_hn_forward_loss_host_submit(
            self.h, C.byref(step), hp(f0), hp(uv), hp(amps), hp(gain), hp(noise_gain), hp(taps_or_bands), hp(w),
            hp(noise), hp(target), slot, self._pipe_loss.data_ptr() + 8 * slot, hp(audio_out)))

    def hn_forward_loss_host_wait(self, slot):
        self.check(self.lib.dgc_hn_forward_loss_host_wait(self.h, slot))
        return float(self._pipe_loss[slot])


_cudart_lib = None


def _cudart():
    """The CUDA runtime torch already loaded (for plain cudaMemcpy of library-owned device tables)."""
    global _cudart_lib
    if _cudart_lib is None:
        import torch  # noqa: F401
        import glob
        cands = glob.glob(os.path.join(os.path.dirname(torch.__file__), "lib", "libcudart*.so*"))
        cands += glob.glob("/usr/local/cuda/lib64/libcudart.so*")
        site = os.path.dirname(os.path.dirname(torch.__file__))
        cands = glob.glob(os.path.join(site, "nvidia", "cuda_runtime", "lib", "libcudart.so*")) + cands
        if not cands:
            raise DgenCudaError("libcudart not found")
        _cudart_lib = C.CDLL(cands[0])
        _cudart_lib.cudaMemcpy.restype = C.c_int
        _cudart_lib.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    return _cudart_lib
