"""ctypes binding of libf8b200.so (the C-ABI kernel library, `include/f8b200.h`).

There is no fallback: if the library is missing or a call fails the caller gets an
exception.  Nothing here runs on the CPU.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libf8b200.so")
_lib: Optional[ctypes.CDLL] = None

BF16, FP16, FP32 = 0, 1, 2
E4M3, E5M2 = 0, 1

_HP_CODE = {torch.bfloat16: BF16, torch.float16: FP16, torch.float32: FP32}
_FP8_CODE = {torch.float8_e4m3fn: E4M3, torch.float8_e5m2: E5M2}
FP8_DTYPE = {E4M3: torch.float8_e4m3fn, E5M2: torch.float8_e5m2}

# every symbol include/f8b200.h declares
EXPORTS = (
    "f8b200_status_string",
    "f8b200_device_check",
    "f8b200_last_cuda_error",
    "f8b200_amax",
    "f8b200_multi_amax",
    "f8b200_amax_to_scale",
    "f8b200_cast",
    "f8b200_cast_dynamic",
    "f8b200_cast_scatter",
    "f8b200_multi_cast",
    "f8b200_transpose_u8",
    "f8b200_delayed_sync",
    "f8b200_gemm_fp8",
    "f8b200_gemm_fp8_ws",
    "f8b200_gemm_fp8_static_scratch",
    "f8b200_gemm_kernel_choice",
    "f8b200_gemm_fp8_scatter_rows",
    "f8b200_sum_slots",
    "f8b200_rmsnorm_amax",
    "f8b200_rmsnorm_cast",
    "f8b200_swiglu_amax",
    "f8b200_swiglu_amax_approx",
    "f8b200_swiglu_cast",
    "f8b200_rmsnorm_bwd_workspace_bytes",
    "f8b200_rmsnorm_bwd",
    "f8b200_swiglu_bwd",
    "f8b200_swiglu_bwd_approx",
    "f8b200_read_device_error",
    "f8b200_check_device_error",
)


class F8B200Error(RuntimeError):
    pass


def lib_path() -> str:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Loads the kernel library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise F8B200Error(
            f"{_LIB_PATH} is missing: build it with `python -m float8_experimental_b200.csrc.build` "
            "(there is no CPU or PyTorch fallback for these kernels)"
        )
    lib = ctypes.CDLL(_LIB_PATH)
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.f8b200_status_string.restype = ctypes.c_char_p
    lib.f8b200_status_string.argtypes = [i32]
    lib.f8b200_last_cuda_error.restype = ctypes.c_char_p
    lib.f8b200_last_cuda_error.argtypes = []
    lib.f8b200_device_check.argtypes = []
    lib.f8b200_amax.argtypes = [vp, i32, i64, vp, vp]
    lib.f8b200_multi_amax.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(i64), i32, i32, vp, vp]
    lib.f8b200_amax_to_scale.argtypes = [vp, i64, i32, i32, i32, vp, vp]
    lib.f8b200_cast.argtypes = [vp, i32, i64, i64, i64, i32, vp, vp, i32, i32, vp, i64, vp, i64, vp, i32, vp]
    lib.f8b200_cast_scatter.argtypes = [vp, i32, i64, i64, i64, i32, vp, vp, i32, i32, ctypes.POINTER(vp), i32, i64,
                                        vp]
    lib.f8b200_cast_dynamic.argtypes = [vp, i32, i64, i64, i32, vp, vp, vp, vp]
    lib.f8b200_multi_cast.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(i64), i32, i32, vp, i32, i32, ctypes.POINTER(vp), vp]
    lib.f8b200_transpose_u8.argtypes = [vp, i64, i64, i64, vp, i64, vp]
    lib.f8b200_delayed_sync.argtypes = [vp, vp, i64, i64, i32, i64, i32, vp, vp, i64, vp]
    lib.f8b200_gemm_fp8.argtypes = [vp, i32, i64, vp, i32, i64, vp, vp, vp, i32, vp, i64, i64, i64, i64, i32, vp]
    lib.f8b200_gemm_fp8_static_scratch.argtypes = lib.f8b200_gemm_fp8.argtypes
    lib.f8b200_gemm_fp8_ws.argtypes = [vp, i32, i32, i64, vp, i32, i32, i64, vp, vp, vp, i32, vp, i64, i64, i64, i64,
                                       i32, vp, i64, vp]
    lib.f8b200_rmsnorm_amax.argtypes = [vp, i32, i64, i64, i64, vp, ctypes.c_float, vp, vp, vp]
    lib.f8b200_rmsnorm_cast.argtypes = [vp, i32, i64, i64, i64, vp, vp, vp, i32, vp, vp, i64, vp]
    lib.f8b200_swiglu_amax.argtypes = [vp, vp, i32, i64, i64, i64, i64, vp, i64, vp, vp]
    lib.f8b200_swiglu_amax_approx.argtypes = [vp, vp, i32, i64, i64, i64, i64, vp, i64, vp, vp]
    lib.f8b200_swiglu_cast.argtypes = [vp, vp, i32, i64, i64, i64, i64, vp, i32, vp, vp, i64, vp]
    lib.f8b200_rmsnorm_bwd_workspace_bytes.argtypes = [i64]
    lib.f8b200_rmsnorm_bwd_workspace_bytes.restype = i64
    lib.f8b200_rmsnorm_bwd.argtypes = [vp, vp, i32, i64, i64, i64, i64, vp, vp, vp, i64, vp, vp, i64, vp]
    lib.f8b200_swiglu_bwd.argtypes = [vp, vp, vp, i32, i64, i64, i64, i64, i64, vp, vp, i64, vp]
    lib.f8b200_swiglu_bwd_approx.argtypes = [vp, vp, vp, i32, i64, i64, i64, i64, i64, vp, vp, i64, vp]
    lib.f8b200_read_device_error.argtypes = [ctypes.POINTER(ctypes.c_uint32)]
    lib.f8b200_check_device_error.argtypes = []
    lib.f8b200_gemm_kernel_choice.argtypes = [i64, i64, i64]
    lib.f8b200_gemm_fp8_scatter_rows.argtypes = [vp, i32, i32, i64, vp, i32, i32, i64, vp, vp, vp, i32, ctypes.POINTER(vp),
                                                 i32, i64, i64, i64, i64, i64, vp, i64, vp]
    lib.f8b200_sum_slots.argtypes = [vp, i32, i64, i32, i64, vp, vp]
    for name in EXPORTS:
        fn = getattr(lib, name)
        if fn.restype is not ctypes.c_char_p and fn.restype is not i64:
            fn.restype = i32
    _lib = lib
    return lib


def _check(status: int, what: str) -> None:
    if status == 0:
        return
    lib = load()
    msg = lib.f8b200_status_string(status).decode()
    detail = lib.f8b200_last_cuda_error().decode() if status == -4 else ""
    raise F8B200Error(f"{what}: {msg}" + (f" [{detail}]" if detail else ""))


def hp_code(dtype: torch.dtype) -> int:
    try:
        return _HP_CODE[dtype]
    except KeyError:
        raise F8B200Error(f"unsupported high-precision dtype {dtype}") from None


def fp8_code(dtype: torch.dtype) -> int:
    try:
        return _FP8_CODE[dtype]
    except KeyError:
        raise F8B200Error(f"unsupported float8 dtype {dtype}") from None


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise F8B200Error("f8b200 kernels run on CUDA tensors only (no CPU path exists)")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# ---------------------------------------------------------------------------
# instrumentation for the benchmark: kernel launch count and, on request, CUDA events
# around every launch (recorded on the launching stream)
# ---------------------------------------------------------------------------
_launches = 0
_events_on = False
_events = {}


def reset_counters() -> None:
    global _launches
    _launches = 0
    _events.clear()


def launch_count() -> int:
    return _launches


def enable_kernel_events(on: bool) -> None:
    global _events_on
    _events_on = bool(on)


def kernel_event_totals():
    """{kind: (total_ms, launches)} of the launches recorded since reset_counters()."""
    torch.cuda.synchronize()
    return {k: (sum(a.elapsed_time(b) for a, b in v), len(v)) for k, v in _events.items()}


class _Launch:
    """Context manager around one kernel launch on `device`: makes that device current
    (only if it is not already), counts the launch, optionally times it."""

    __slots__ = ("kind", "n", "start", "guard")

    def __init__(self, kind: str, device: torch.device, n: int = 1):
        self.kind, self.n, self.start = kind, n, None
        idx = device.index
        self.guard = None if (idx is None or idx == torch.cuda.current_device()) else torch.cuda.device(idx)

    def __enter__(self):
        global _launches
        _launches += self.n
        if self.guard is not None:
            self.guard.__enter__()
        if _events_on:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if self.start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            _events.setdefault(self.kind, []).append((self.start, end))
        if self.guard is not None:
            self.guard.__exit__(*exc)
        return False


# ---------------------------------------------------------------------------
# thin tensor-level wrappers (each sets the device of its first argument)
# ---------------------------------------------------------------------------
def amax(x: torch.Tensor, out: torch.Tensor) -> None:
    _require_cuda(x, out)
    with _Launch("amax", x.device):
        _check(load().f8b200_amax(x.data_ptr(), hp_code(x.dtype), x.numel(), out.data_ptr(), _stream(x)), "f8b200_amax")


def multi_amax(xs: Sequence[torch.Tensor], out: torch.Tensor) -> None:
    n = len(xs)
    if n == 0:
        return
    _require_cuda(out, *xs)
    dt = xs[0].dtype
    if any(t.dtype != dt for t in xs):
        raise F8B200Error("multi_amax needs tensors of one dtype")
    ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in xs])
    numels = (ctypes.c_int64 * n)(*[t.numel() for t in xs])
    with _Launch("amax", out.device, (n + 127) // 128):
        _check(load().f8b200_multi_amax(ptrs, numels, n, hp_code(dt), out.data_ptr(), _stream(out)), "f8b200_multi_amax")


def amax_to_scale(amax_t: torch.Tensor, fp8_kind: int, amax_dtype: int, orig_dtype: int, out: torch.Tensor) -> None:
    _require_cuda(amax_t, out)
    with _Launch("scale", out.device):
        _check(
            load().f8b200_amax_to_scale(amax_t.data_ptr(), amax_t.numel(), fp8_kind, amax_dtype, orig_dtype,
                                        out.data_ptr(), _stream(out)),
            "f8b200_amax_to_scale",
        )


def cast(x: torch.Tensor, rows: int, cols: int, ld_x: int, scale_src: int, scale_in: torch.Tensor,
         scale_out: Optional[torch.Tensor], product_fp32: bool, fp8_kind: int, out: Optional[torch.Tensor],
         ld_out: int, out_t: Optional[torch.Tensor], ld_out_t: int, amax_out: Optional[torch.Tensor],
         reverse: bool) -> None:
    _require_cuda(x, scale_in, scale_out, out, out_t, amax_out)
    with _Launch("cast", x.device):
        _check(
            load().f8b200_cast(x.data_ptr(), hp_code(x.dtype), rows, cols, ld_x, scale_src, scale_in.data_ptr(),
                               _ptr(scale_out), int(product_fp32), fp8_kind, _ptr(out), ld_out, _ptr(out_t),
                               ld_out_t, _ptr(amax_out), int(reverse), _stream(x)),
            "f8b200_cast",
        )


def cast_dynamic(x: torch.Tensor, rows: int, cols: int, fp8_kind: int, amax_out: torch.Tensor, scale_out: torch.Tensor,
                 out: torch.Tensor) -> None:
    """`f8b200_cast_dynamic`: amax + cast of a contiguous matrix in one host call (two launches)."""
    _require_cuda(x, amax_out, scale_out, out)
    with _Launch("cast", x.device, 2):
        _check(load().f8b200_cast_dynamic(x.data_ptr(), hp_code(x.dtype), rows, cols, fp8_kind, amax_out.data_ptr(),
                                          scale_out.data_ptr(), out.data_ptr(), _stream(x)), "f8b200_cast_dynamic")


def multi_cast(xs: Sequence[torch.Tensor], scales: torch.Tensor, product_fp32: bool, fp8_kind: int,
               outs: Sequence[torch.Tensor]) -> None:
    """`f8b200_multi_cast`: every contiguous tensor of `xs` cast with its own scale (`scales[i]`) into
    `outs[i]`, one launch per 96 tensors."""
    n = len(xs)
    if n == 0:
        return
    _require_cuda(scales, *xs, *outs)
    dt = xs[0].dtype
    if any(t.dtype != dt for t in xs):
        raise F8B200Error("multi_cast needs tensors of one dtype")
    ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in xs])
    optrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in outs])
    numels = (ctypes.c_int64 * n)(*[t.numel() for t in xs])
    with _Launch("cast", scales.device, (n + 95) // 96):
        _check(load().f8b200_multi_cast(ptrs, numels, n, hp_code(dt), scales.data_ptr(), int(product_fp32), fp8_kind,
                                        optrs, _stream(scales)), "f8b200_multi_cast")


def transpose_u8(src: torch.Tensor, rows: int, cols: int, ld_in: int, dst: torch.Tensor, ld_out: int) -> None:
    _require_cuda(src, dst)
    with _Launch("transpose", src.device):
        _check(load().f8b200_transpose_u8(src.data_ptr(), rows, cols, ld_in, dst.data_ptr(), ld_out, _stream(src)),
               "f8b200_transpose_u8")


def delayed_sync(amax_t: torch.Tensor, hist: torch.Tensor, n_e4m3: int, orig_dtype: int, scale_out: torch.Tensor,
                 hist_out: Optional[torch.Tensor]) -> None:
    _require_cuda(amax_t, hist, scale_out, hist_out)
    rows, hist_len = hist.shape
    with _Launch("sync", hist.device):
        _check(
            load().f8b200_delayed_sync(amax_t.data_ptr(), hist.data_ptr(), hist.stride(0), rows, hist_len, n_e4m3,
                                       orig_dtype, scale_out.data_ptr(), _ptr(hist_out),
                                       hist_out.stride(0) if hist_out is not None else 0, _stream(hist)),
            "f8b200_delayed_sync",
        )


# ---------------------------------------------------------------------------
# optional single-GPU library: the cluster-multicast GEMM (csrc/gemm_mc.cu).  Runs on several GPUs
# ship without it; everything then goes through libf8b200.so.
# ---------------------------------------------------------------------------
_MC_LIB_PATH = os.path.join(os.path.dirname(_LIB_PATH), "libf8b200_mc.so")
_mc_lib = None
_mc_tried = False


def load_mc():
    """The multicast GEMM library, or None when it was not built / not shipped."""
    global _mc_lib, _mc_tried
    if not _mc_tried:
        _mc_tried = True
        if os.path.exists(_MC_LIB_PATH):
            lib = ctypes.CDLL(_MC_LIB_PATH)
            vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
            lib.f8b200_mc_gemm_fp8.argtypes = [vp, i32, i32, i64, vp, i32, i32, i64, vp, vp, vp, i32, vp, i64, i64, i64,
                                               i64, i32, i32, vp, i64, vp]
            lib.f8b200_mc_gemm_fp8.restype = i32
            lib.f8b200_mc_read_device_error.argtypes = [ctypes.POINTER(ctypes.c_uint32)]
            lib.f8b200_mc_read_device_error.restype = i32
            _mc_lib = lib
    return _mc_lib


def _single_gpu_job() -> bool:
    """True only when this process can be sure it belongs to a job that uses ONE GPU: exactly one
    CUDA device is visible, no launcher announced more than one rank (WORLD_SIZE /
    LOCAL_WORLD_SIZE, which are set before `init_process_group` runs), and no process group with
    more than one rank exists.  The multicast GEMM may run in such jobs only: its TMA loads must
    never be handed memory of another GPU."""
    if torch.cuda.device_count() != 1:
        return False
    for var in ("WORLD_SIZE", "LOCAL_WORLD_SIZE"):
        try:
            if int(os.environ.get(var, "1")) > 1:
                return False
        except ValueError:
            return False
    if torch.distributed.is_available() and torch.distributed.is_initialized() and torch.distributed.get_world_size() > 1:
        return False
    return True


def _mc_cluster(m: int, n: int, k: int):
    """Cluster shape (tiles along M, along N) of the multicast GEMM for this product, or None
    to use the kernels of libf8b200.so.  Opt-in: F8B200_GEMM_MC=21 / 22 / 41 select 2 x 1 or
    2 x 2 clusters of 256x256 tiles, or two CTA pairs sharing B; by default (and with
    F8B200_GEMM_MC=0, or when F8B200_GEMM_MODE forces a kernel) nothing uses it, because the
    512x256 pair kernel of libf8b200.so measured faster on every product.  Only jobs on a single
    GPU may use it at all (`_single_gpu_job`; the C entry point checks on its side that every
    pointer is the current device's own memory)."""
    mode = os.environ.get("F8B200_GEMM_MC", "0")
    if mode not in ("21", "22", "41") or not _single_gpu_job() or load_mc() is None:
        return None
    if os.environ.get("F8B200_GEMM_MODE", "")[:1] in ("1", "2", "w", "p"):
        return None
    return {"21": (2, 1), "22": (2, 2), "41": (4, 1)}[mode]


GEMM_WORKSPACE_BYTES = 256  # F8B200_GEMM_WORKSPACE_BYTES in include/f8b200.h
_gemm_workspaces: dict = {}


def _gemm_workspace(device: torch.device, stream: int) -> torch.Tensor:
    """Scheduling workspace of the GEMMs issued on `stream` of `device`: one small buffer per
    stream, kept for the life of the process, because GEMMs that may overlap must not share one."""
    key = (device.index, stream)
    ws = _gemm_workspaces.get(key)
    if ws is None:
        ws = torch.empty(GEMM_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        _gemm_workspaces[key] = ws
    return ws


def gemm_fp8(a: torch.Tensor, lda: int, b: torch.Tensor, ldb: int, scale_a: torch.Tensor, scale_b: torch.Tensor,
             bias: Optional[torch.Tensor], out: torch.Tensor, ldo: int, m: int, n: int, k: int,
             use_fast_accum: bool, a_mn_major: bool = False, b_mn_major: bool = False) -> None:
    """`f8b200_gemm_fp8_ws` with this stream's workspace (dynamic tile scheduling).  `a` is the
    [m, k] operand stored K-contiguous, or with `a_mn_major` its transpose stored [k, m]; likewise
    `b` ([n, k], or [k, n] with `b_mn_major`).  F8B200_GEMM_WS=0 in the environment selects the
    workspace-free `f8b200_gemm_fp8` (K-major operands only)."""
    _require_cuda(a, b, scale_a, scale_b, bias, out)
    stream = _stream(a)
    cluster = _mc_cluster(m, n, k)
    with _Launch("gemm", a.device):
        if cluster is not None:
            ws = _gemm_workspace(a.device, stream)
            rc = _mc_lib.f8b200_mc_gemm_fp8(a.data_ptr(), fp8_code(a.dtype), int(a_mn_major), lda, b.data_ptr(),
                                            fp8_code(b.dtype), int(b_mn_major), ldb, scale_a.data_ptr(),
                                            scale_b.data_ptr(), _ptr(bias), hp_code(out.dtype), out.data_ptr(), ldo,
                                            m, n, k, cluster[0], cluster[1], ws.data_ptr(), ws.numel(), stream)
            if rc != -6:  # F8B200_ERR_UNSUPPORTED: such clusters cannot be scheduled here / layout not covered
                if rc != 0:
                    raise F8B200Error(f"f8b200_mc_gemm_fp8: {load().f8b200_status_string(rc).decode()}")
                return
        if os.environ.get("F8B200_GEMM_WS", "1") == "0" and not (a_mn_major or b_mn_major):
            _check(
                load().f8b200_gemm_fp8(a.data_ptr(), fp8_code(a.dtype), lda, b.data_ptr(), fp8_code(b.dtype), ldb,
                                       scale_a.data_ptr(), scale_b.data_ptr(), _ptr(bias), hp_code(out.dtype),
                                       out.data_ptr(), ldo, m, n, k, int(use_fast_accum), stream),
                "f8b200_gemm_fp8",
            )
        else:
            ws = _gemm_workspace(a.device, stream)
            _check(
                load().f8b200_gemm_fp8_ws(a.data_ptr(), fp8_code(a.dtype), int(a_mn_major), lda, b.data_ptr(),
                                          fp8_code(b.dtype), int(b_mn_major), ldb, scale_a.data_ptr(),
                                          scale_b.data_ptr(), _ptr(bias), hp_code(out.dtype), out.data_ptr(), ldo, m,
                                          n, k, int(use_fast_accum), ws.data_ptr(), ws.numel(), stream),
                "f8b200_gemm_fp8_ws",
            )


def gemm_fp8_scatter_rows(a: torch.Tensor, lda: int, b: torch.Tensor, ldb: int, scale_a: torch.Tensor,
                          scale_b: torch.Tensor, out_dtype: torch.dtype, out_ptrs: Sequence[int], rows_per_block: int,
                          ldo: int, m: int, n: int, k: int, a_mn_major: bool = False, b_mn_major: bool = False) -> None:
    """`f8b200_gemm_fp8_scatter_rows`: the GEMM whose output row blocks go round-robin to the
    addresses in `out_ptrs` (this device's own buffer and peer-mapped buffers of other devices)."""
    _require_cuda(a, b, scale_a, scale_b)
    stream = _stream(a)
    ws = _gemm_workspace(a.device, stream)
    arr = (ctypes.c_void_p * len(out_ptrs))(*[ctypes.c_void_p(p) for p in out_ptrs])
    with _Launch("gemm", a.device):
        _check(
            load().f8b200_gemm_fp8_scatter_rows(a.data_ptr(), fp8_code(a.dtype), int(a_mn_major), lda, b.data_ptr(),
                                                fp8_code(b.dtype), int(b_mn_major), ldb, scale_a.data_ptr(),
                                                scale_b.data_ptr(), None, hp_code(out_dtype), arr, len(out_ptrs),
                                                rows_per_block, ldo, m, n, k, ws.data_ptr(), ws.numel(), stream),
            "f8b200_gemm_fp8_scatter_rows",
        )


def sum_slots(slots: torch.Tensor, n_slots: int, slot_stride: int, numel: int, out: torch.Tensor) -> None:
    """`f8b200_sum_slots`: out = sum of the first `n_slots` slots of `slots` (fp32 accumulation)."""
    _require_cuda(slots, out)
    with _Launch("sum_slots", out.device):
        _check(
            load().f8b200_sum_slots(slots.data_ptr(), n_slots, slot_stride, hp_code(out.dtype), numel, out.data_ptr(),
                                    _stream(out)),
            "f8b200_sum_slots",
        )


def gemm_kernel_choice(m: int, n: int, k: int) -> int:
    """Code of the kernel the library would run for this product (see include/f8b200.h)."""
    return int(load().f8b200_gemm_kernel_choice(m, n, k))


def gemm_fp8_static_scratch(a: torch.Tensor, lda: int, b: torch.Tensor, ldb: int, scale_a: torch.Tensor,
                            scale_b: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, ldo: int, m: int,
                            n: int, k: int, use_fast_accum: bool) -> None:
    """`f8b200_gemm_fp8_static_scratch`: dynamic tile scheduling with the scheduling words in the
    library's own static device array (at most 16 streams per device)."""
    _require_cuda(a, b, scale_a, scale_b, bias, out)
    with _Launch("gemm", a.device):
        _check(
            load().f8b200_gemm_fp8_static_scratch(a.data_ptr(), fp8_code(a.dtype), lda, b.data_ptr(),
                                                  fp8_code(b.dtype), ldb, scale_a.data_ptr(), scale_b.data_ptr(),
                                                  _ptr(bias), hp_code(out.dtype), out.data_ptr(), ldo, m, n, k,
                                                  int(use_fast_accum), _stream(a)),
            "f8b200_gemm_fp8_static_scratch",
        )


def rmsnorm_amax(x: torch.Tensor, rows: int, cols: int, ld: int, weight: torch.Tensor, eps: float,
                 rstd_out: torch.Tensor, amax_out: torch.Tensor) -> None:
    _require_cuda(x, weight, rstd_out, amax_out)
    with _Launch("norm_amax", x.device):
        _check(
            load().f8b200_rmsnorm_amax(x.data_ptr(), hp_code(x.dtype), rows, cols, ld, weight.data_ptr(), float(eps),
                                       rstd_out.data_ptr(), amax_out.data_ptr(), _stream(x)),
            "f8b200_rmsnorm_amax",
        )


def rmsnorm_cast(x: torch.Tensor, rows: int, cols: int, ld: int, weight: torch.Tensor, rstd: torch.Tensor,
                 amax: torch.Tensor, scale_out: Optional[torch.Tensor], out: torch.Tensor, ld_out: int) -> None:
    _require_cuda(x, weight, rstd, amax, scale_out, out)
    with _Launch("norm_cast", x.device):
        _check(
            load().f8b200_rmsnorm_cast(x.data_ptr(), hp_code(x.dtype), rows, cols, ld, weight.data_ptr(),
                                       rstd.data_ptr(), amax.data_ptr(), fp8_code(out.dtype), _ptr(scale_out),
                                       out.data_ptr(), ld_out, _stream(x)),
            "f8b200_rmsnorm_cast",
        )


def swiglu_amax(a: torch.Tensor, b: torch.Tensor, rows: int, cols: int, ld_a: int, ld_b: int,
                y_out: Optional[torch.Tensor], ld_y: int, amax_out: torch.Tensor, approx: bool = False) -> None:
    _require_cuda(a, b, y_out, amax_out)
    args = (a.data_ptr(), b.data_ptr(), hp_code(a.dtype), rows, cols, ld_a, ld_b, _ptr(y_out), ld_y,
            amax_out.data_ptr(), _stream(a))
    with _Launch("glu_amax", a.device):
        if approx:
            _check(load().f8b200_swiglu_amax_approx(*args), "f8b200_swiglu_amax_approx")
        else:
            _check(load().f8b200_swiglu_amax(*args), "f8b200_swiglu_amax")


def swiglu_cast(a: torch.Tensor, b: torch.Tensor, rows: int, cols: int, ld_a: int, ld_b: int, amax: torch.Tensor,
                scale_out: Optional[torch.Tensor], out: torch.Tensor, ld_out: int) -> None:
    _require_cuda(a, b, amax, scale_out, out)
    with _Launch("glu_cast", a.device):
        _check(
            load().f8b200_swiglu_cast(a.data_ptr(), b.data_ptr(), hp_code(a.dtype), rows, cols, ld_a, ld_b,
                                      amax.data_ptr(), fp8_code(out.dtype), _ptr(scale_out), out.data_ptr(), ld_out,
                                      _stream(a)),
            "f8b200_swiglu_cast",
        )


def cast_scatter(x: torch.Tensor, rows: int, cols: int, ld_x: int, amax: torch.Tensor, scale_out: torch.Tensor,
                 fp8_kind: int, out_ptrs: Sequence[int], ld_out: int) -> None:
    """Dynamic cast of `x` whose row-major bytes go to every address in `out_ptrs` (this
    device's own buffer and peer-mapped buffers of other devices)."""
    _require_cuda(x, amax, scale_out)
    arr = (ctypes.c_void_p * len(out_ptrs))(*[ctypes.c_void_p(p) for p in out_ptrs])
    with _Launch("cast", x.device):
        _check(
            load().f8b200_cast_scatter(x.data_ptr(), hp_code(x.dtype), rows, cols, ld_x, 1, amax.data_ptr(),
                                       scale_out.data_ptr(), 0, fp8_kind, arr, len(out_ptrs), ld_out, _stream(x)),
            "f8b200_cast_scatter",
        )


def rmsnorm_bwd(x: torch.Tensor, g: torch.Tensor, rows: int, cols: int, ld_x: int, ld_g: int, weight: torch.Tensor,
                rstd: torch.Tensor, dx: torch.Tensor, dweight: torch.Tensor) -> None:
    _require_cuda(x, g, weight, rstd, dx, dweight)
    nbytes = int(load().f8b200_rmsnorm_bwd_workspace_bytes(cols))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    with _Launch("norm_bwd", x.device, 2):
        _check(
            load().f8b200_rmsnorm_bwd(x.data_ptr(), g.data_ptr(), hp_code(x.dtype), rows, cols, ld_x, ld_g,
                                      weight.data_ptr(), rstd.data_ptr(), dx.data_ptr(), cols, dweight.data_ptr(),
                                      ws.data_ptr(), nbytes, _stream(x)),
            "f8b200_rmsnorm_bwd",
        )


def swiglu_bwd(a: torch.Tensor, b: torch.Tensor, g: torch.Tensor, rows: int, cols: int, ld_a: int, ld_b: int,
               ld_g: int, da: torch.Tensor, db: torch.Tensor, approx: bool = False) -> None:
    _require_cuda(a, b, g, da, db)
    args = (a.data_ptr(), b.data_ptr(), g.data_ptr(), hp_code(a.dtype), rows, cols, ld_a, ld_b, ld_g, da.data_ptr(),
            db.data_ptr(), cols, _stream(a))
    with _Launch("glu_bwd", a.device):
        if approx:
            _check(load().f8b200_swiglu_bwd_approx(*args), "f8b200_swiglu_bwd_approx")
        else:
            _check(load().f8b200_swiglu_bwd(*args), "f8b200_swiglu_bwd")


def check_device_error() -> None:
    """Raises F8B200Error (F8B200_ERR_TIMEOUT) when a bounded wait inside a GEMM kernel gave up
    since the last poll: the outputs of those launches are undefined.  Synchronises the device, so
    call it where the program synchronises anyway (the end of a step, a benchmark's timed region).
    With F8B200_POLL_ERRORS=1 in the environment `sync_float8_amax_and_scale_history` and
    `precompute_float8_dynamic_scale_for_fsdp` poll it once per call."""
    flags = read_device_error()
    if flags != 0:
        raise F8B200Error(f"device error word {flags:#x}: " + load().f8b200_status_string(-7).decode())


def poll_errors_if_enabled() -> None:
    if os.environ.get("F8B200_POLL_ERRORS", "0") == "1" and torch.cuda.is_available():
        check_device_error()


def read_device_error() -> int:
    v = ctypes.c_uint32(0)
    _check(load().f8b200_read_device_error(ctypes.byref(v)), "f8b200_read_device_error")
    flags = int(v.value)
    if _mc_lib is not None:  # the multicast library keeps an error word of its own
        w = ctypes.c_uint32(0)
        if _mc_lib.f8b200_mc_read_device_error(ctypes.byref(w)) == 0:
            flags |= int(w.value)
    return flags
