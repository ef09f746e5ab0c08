"""ctypes binding of ``libdionw_b200.so`` (the C ABI in ``include/dionw_b200.h``).

The library is the only implementation of the step: when it is missing or a
call fails this module raises, it never falls back to another path.  Wrappers
take torch tensors, check nothing but what the C side cannot, and launch on the
current CUDA stream of the tensors' device.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint8, c_void_p
from pathlib import Path
from typing import Sequence

import torch
from torch import Tensor

LIBRARY_PATH = Path(__file__).resolve().parent / "lib" / "libdionw_b200.so"

F32, F16, BF16 = 0, 1, 2
NS_GRAM, NS_POLAR_EXPRESS, NS_KELLER, NS_GRAM_FULL = 0, 1, 2, 3
_DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

_ERRORS = {
    -1: ValueError,
    -2: RuntimeError,
    -3: RuntimeError,
    -4: NotImplementedError,
    -5: RuntimeError,
    -6: RuntimeError,
}

_PP = POINTER(c_void_p)
_I64P = POINTER(c_int64)

# name -> (restype, argtypes); mirrors include/dionw_b200.h one to one.
SIGNATURES: dict[str, tuple[object, tuple[object, ...]]] = {
    "dionw_last_error": (None, (ctypes.c_char_p, c_size_t)),
    "dionw_version": (c_char_p, ()),
    "dionw_device_status": (c_int, (POINTER(c_int),)),
    "dionw_launch_count": (c_int64, ()),
    "dionw_check_device": (c_int, ()),
    "dionw_gemm_dynamic_tiles": (c_int, (c_int,)),
    "dionw_selftest_wait_timeout": (c_int, (c_int64, c_void_p, c_void_p)),
    "dionw_accumulate_row_l1_run": (c_int, (_PP, c_int, _I64P, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p)),
    "dionw_accumulate_copy_decay_run": (
        c_int, (_PP, c_int, _I64P, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_int, c_void_p)),
    "dionw_select_rows": (c_int, (c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p)),
    "dionw_block_norms": (c_int, (c_void_p, c_int64, c_int64, c_void_p, c_void_p)),
    "dionw_pack_rows": (
        c_int, (c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_float, c_float,
                c_void_p, c_int, c_int64, c_void_p)),
    "dionw_transpose_2byte": (c_int, (c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p)),
    "dionw_newton_schulz_workspace_bytes": (c_size_t, (c_int64, c_int64, c_int64, c_int)),
    "dionw_newton_schulz": (
        c_int, (c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p, c_size_t, c_void_p, c_void_p)),
    "dionw_newton_schulz_rowsq_parts": (c_int64, (c_int64,)),
    "dionw_newton_schulz_static": (
        c_int, (c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p)),
    "dionw_symmetric_product": (
        c_int, (c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64, c_float, c_float,
                c_void_p, c_int64, c_void_p, c_float, c_int, c_void_p)),
    "dionw_batched_gemm": (
        c_int, (c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_int64, c_float, c_void_p, c_int64, c_int64,
                c_int64, c_int64, c_int64, c_int, c_int, c_void_p)),
    "dionw_row_sumsq_bf16": (c_int, (c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p)),
    "dionw_normuon_rows": (
        c_int, (c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_float, c_float, c_float,
                c_void_p, c_int, c_void_p, c_void_p, c_void_p)),
    "dionw_apply_round": (
        c_int, (_PP, _I64P, _PP, _PP, _PP, _PP, c_int, c_int64, c_int64, c_int64, c_int64, c_float, c_void_p, c_int,
                c_int, c_void_p, c_void_p)),
    "dionw_decay_job_bytes": (c_size_t, ()),
    "dionw_decay_job_begin": (
        c_int, (c_void_p, _PP, _PP, _I64P, c_int, c_int64, c_int64, c_float, c_void_p, c_int, c_void_p)),
    "dionw_gemm_side_job": (None, (c_void_p,)),
    "dionw_write_scalars": (c_int, (c_void_p, POINTER(c_float), c_int64, c_void_p)),
    "dionw_apply_run": (
        c_int, (_PP, _I64P, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                c_float, c_int, c_void_p)),
    "dionw_adamw_multi": (
        c_int, (_PP, _PP, _PP, _PP, _PP, _I64P, c_int, c_float, c_float, c_float, c_float, c_float, c_void_p,
                c_void_p)),
    "dionw_ema_multi": (c_int, (_PP, _PP, _I64P, c_int, c_int, c_float, c_int, c_void_p)),
    "dionw_ema_stage_pack": (c_int, (_PP, _I64P, _I64P, c_int, c_int, c_void_p, c_void_p)),
    "dionw_cpu_ema_job_start": (c_void_p, (_PP, _PP, _I64P, POINTER(c_uint8), c_int, c_float, c_void_p, c_int)),
    "dionw_cpu_ema_job_wait_copy": (c_int, (c_void_p,)),
    "dionw_cpu_ema_job_wait_update": (c_int, (c_void_p,)),
    "dionw_cpu_ema_job_done": (c_int, (c_void_p,)),
    "dionw_cpu_ema_job_destroy": (None, (c_void_p,)),
}

_lib: ctypes.CDLL | None = None


def library() -> ctypes.CDLL:
    """Load the shared library (once).

    Raises:
        RuntimeError: If it has not been built; there is no other implementation.
    """
    global _lib
    if _lib is None:
        if not LIBRARY_PATH.exists():
            raise RuntimeError(
                f"{LIBRARY_PATH} is missing: build it with `python -m dionw_b200.build_ext` "
                "(needs nvcc). dionw_b200 has no fallback path."
            )
        lib = ctypes.CDLL(str(LIBRARY_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = list(argtypes)
        _lib = lib
    return _lib


def last_error() -> str:
    buffer = ctypes.create_string_buffer(512)
    library().dionw_last_error(buffer, 512)
    return buffer.value.decode(errors="replace")


def _check(status: int) -> None:
    if status != 0:
        raise _ERRORS.get(status, RuntimeError)(f"dionw_b200: {last_error()} (code {status})")


def _stream(t: Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _ptr_array(tensors: Sequence[Tensor]):
    return (c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _i64_array(values: Sequence[int]):
    return (c_int64 * len(values))(*values)


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"dionw_b200 kernels take float32, float16 or bfloat16, got {dtype}") from None


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(library().dionw_launch_count())


def device_status() -> int:
    """Read and clear the device status word (synchronises)."""
    value = c_int(0)
    _check(library().dionw_device_status(ctypes.byref(value)))
    return value.value


class DeviceWaitError(RuntimeError):
    """A bounded wait inside a kernel ran out (``DIONW_ERR_DEVICE_WAIT``)."""


def check_device() -> None:
    """Synchronise the current device and raise if a kernel's bounded wait ran out since the last check.

    Raises:
        DeviceWaitError: The device status word was non-zero (it is cleared by the read).
    """
    status = library().dionw_check_device()
    if status == -5:
        raise DeviceWaitError(f"dionw_b200: {last_error()} (code {status})")
    _check(status)


def gemm_dynamic_tiles(on: bool | None = None) -> bool:
    """Set (or with None only read) whether multi-wave tensor-core products draw their tiles from a
    device counter instead of a fixed stride; returns the previous setting.  Process-wide."""
    return bool(library().dionw_gemm_dynamic_tiles(-1 if on is None else int(on)))


def selftest_wait_timeout(limit_us: int, gave_up: Tensor) -> None:
    """Launch the wait self-test on ``gave_up``'s device: a kernel that waits ``limit_us`` on a
    barrier nothing arrives on, gives up and sets ``gave_up`` (int32 scalar) to 1."""
    _check(library().dionw_selftest_wait_timeout(limit_us, gave_up.data_ptr(), _stream(gave_up)))


# ---------------------------------------------------------------------------
# momentum passes
# ---------------------------------------------------------------------------
def accumulate_row_l1_run(grads: Sequence[Tensor], rows_per_tensor: Sequence[int], momentum: Tensor,
                          scores: Tensor, sumsq: Tensor, cols: int) -> None:
    code = dtype_code(grads[0].dtype)
    _check(library().dionw_accumulate_row_l1_run(
        _ptr_array(grads), code, _i64_array(rows_per_tensor), len(grads), momentum.data_ptr(),
        scores.data_ptr(), sumsq.data_ptr(), cols, _stream(momentum)))


def accumulate_copy_decay_run(grads: Sequence[Tensor], rows_per_tensor: Sequence[int], momentum: Tensor,
                              out: Tensor, sumsq: Tensor, cols: int, decay: float, nesterov: bool) -> None:
    code = dtype_code(grads[0].dtype)
    _check(library().dionw_accumulate_copy_decay_run(
        _ptr_array(grads), code, _i64_array(rows_per_tensor), len(grads), momentum.data_ptr(),
        out.data_ptr(), sumsq.data_ptr(), cols, decay, int(nesterov), _stream(momentum)))


def select_rows(scores: Tensor, sumsq: Tensor, k: int, index: Tensor, rowmap: Tensor, frob: Tensor) -> None:
    blocks, rows = scores.shape
    _check(library().dionw_select_rows(scores.data_ptr(), sumsq.data_ptr(), blocks, rows, k, index.data_ptr(),
                                       rowmap.data_ptr(), frob.data_ptr(), _stream(scores)))


def block_norms(sumsq: Tensor, frob: Tensor) -> None:
    blocks, rows = sumsq.shape
    _check(library().dionw_block_norms(sumsq.data_ptr(), blocks, rows, frob.data_ptr(), _stream(sumsq)))


def pack_rows(src: Tensor, index: Tensor | None, frob: Tensor, k: int, x: Tensor, *, decay: float,
              decay_rows: bool, eps: float, norm_scale: float = 1.0) -> None:
    blocks, rows, cols = src.shape
    _check(library().dionw_pack_rows(src.data_ptr(), _ptr(index), frob.data_ptr(), blocks, rows, k, cols, decay,
                                     int(decay_rows), eps, norm_scale, x.data_ptr(), dtype_code(x.dtype),
                                     x.stride(-2), _stream(src)))


def transpose_2byte(src: Tensor, dst: Tensor) -> None:
    blocks, rows, cols = src.shape
    _check(library().dionw_transpose_2byte(src.data_ptr(), dst.data_ptr(), blocks, rows, cols, src.stride(-2),
                                           dst.stride(-2), _stream(src)))


# ---------------------------------------------------------------------------
# Newton-Schulz
# ---------------------------------------------------------------------------
def newton_schulz_workspace_bytes(blocks: int, m: int, n: int, kind: int) -> int:
    return int(library().dionw_newton_schulz_workspace_bytes(blocks, m, n, kind))


def newton_schulz_rowsq_parts(n: int) -> int:
    """Partial sums per output row that ``newton_schulz`` writes into ``rowsq`` for ``n`` columns."""
    return int(library().dionw_newton_schulz_rowsq_parts(n))


def newton_schulz(x: Tensor, out: Tensor, m: int, n: int, kind: int, workspace: Tensor,
                  rowsq: Tensor | None = None) -> None:
    """``x``: ``[blocks, m, ldx]`` fp16/bf16 wide operand (overwritten); ``out`` bf16, may alias ``x``.
    ``rowsq`` (fp32 ``[blocks * m, newton_schulz_rowsq_parts(n)]``): partial row sums of ``out**2``."""
    _check(library().dionw_newton_schulz(x.data_ptr(), out.data_ptr(), x.shape[0], m, n, x.stride(-2), kind,
                                         workspace.data_ptr(), workspace.numel() * workspace.element_size(),
                                         _ptr(rowsq), _stream(x)))


STATIC_SCRATCH_BYTES = 64 << 20


def newton_schulz_static(x: Tensor, out: Tensor, m: int, n: int, kind: int) -> None:
    """``newton_schulz`` on the library's built-in 64 MiB scratch: no workspace argument, no
    allocation.  Larger problems raise; calls that overlap on one GPU race on the scratch."""
    _check(library().dionw_newton_schulz_static(x.data_ptr(), out.data_ptr(), x.shape[0], m, n, x.stride(-2),
                                                kind, _stream(x)))


def symmetric_product(a: Tensor, out: Tensor, *, b: Tensor | None = None, cin: Tensor | None = None,
                      alpha: float = 1.0, beta: float = 0.0, out2: Tensor | None = None, diag: float = 0.0) -> None:
    blocks, m, kdim = a.shape
    _check(library().dionw_symmetric_product(
        a.data_ptr(), _ptr(b), blocks, m, kdim, a.stride(-2), 0 if b is None else b.stride(-2), _ptr(cin),
        0 if cin is None else cin.stride(-2), alpha, beta,
        out.data_ptr(), out.stride(-2), _ptr(out2), diag, dtype_code(a.dtype), _stream(a)))


def batched_gemm(a: Tensor, b: Tensor, out: Tensor, *, b_is_nk: bool, cin: Tensor | None = None,
                 beta: float = 0.0) -> None:
    blocks, m, kdim = a.shape
    n = b.shape[1] if b_is_nk else b.shape[2]
    _check(library().dionw_batched_gemm(
        a.data_ptr(), a.stride(-2), b.data_ptr(), b.stride(-2), int(b_is_nk), _ptr(cin),
        0 if cin is None else cin.stride(-2), beta, out.data_ptr(), out.stride(-2), blocks, m, n, kdim,
        dtype_code(a.dtype), dtype_code(out.dtype), _stream(a)))


# ---------------------------------------------------------------------------
# NorMuon and apply
# ---------------------------------------------------------------------------
def row_sumsq_bf16(o: Tensor, cols: int, s: Tensor) -> None:
    blocks, k, _ = o.shape
    _check(library().dionw_row_sumsq_bf16(o.data_ptr(), blocks, k, cols, o.stride(-2), s.data_ptr(), _stream(o)))


def normuon_rows(s: Tensor, variance: Tensor, index: Tensor | None, *, blocks: int, rows: int, k: int, cols: int,
                 weight: float, eps: float, step: float, normalize: bool, denom: Tensor, scale: Tensor,
                 parts: int = 1, step_device: Tensor | None = None) -> None:
    """``s`` holds ``parts`` partial sums per row; ``step_device`` (one fp32 on the device) overrides ``step``."""
    _check(library().dionw_normuon_rows(s.data_ptr(), parts, variance.data_ptr(), _ptr(index), blocks, rows, k, cols,
                                        weight, eps, step, _ptr(step_device), int(normalize), denom.data_ptr(),
                                        scale.data_ptr(), _stream(s)))


def apply_run(weights: Sequence[Tensor], rows_per_tensor: Sequence[int], o: Tensor, rowmap: Tensor | None,
              denom: Tensor, scale: Tensor, *, rows: int, k: int, cols: int, decay_factor: float,
              has_decay: bool) -> None:
    _check(library().dionw_apply_run(
        _ptr_array(weights), _i64_array(rows_per_tensor), len(weights), o.data_ptr(), o.stride(-2), _ptr(rowmap),
        denom.data_ptr(), scale.data_ptr(), rows, k, cols, decay_factor, int(has_decay), _stream(o)))


def apply_round(weights: Sequence[Tensor], rows_per_tensor: Sequence[int], o: Sequence[int],
                rowmap: Sequence[int] | None, denom: Sequence[int], scale: Sequence[int], *, ldo: int,
                rows: int, k: int, cols: int, decay_factor: float, has_decay: bool,
                decay_device: Tensor | None = None, cta_warps: int = 0, decay_job: Tensor | None = None) -> None:
    """The weight update of tensors whose update rows lie in different buffers, in one launch:
    ``o[i]``, ``rowmap[i]``, ``denom[i]``, ``scale[i]`` are the device addresses of the first block
    of tensor ``i`` (bf16 rows, int32 row map, fp32 divisors, fp32 block scales)."""
    n = len(weights)
    _check(library().dionw_apply_round(
        _ptr_array(weights), _i64_array(rows_per_tensor), (c_void_p * n)(*o),
        None if rowmap is None else (c_void_p * n)(*rowmap), (c_void_p * n)(*denom), (c_void_p * n)(*scale), n, ldo,
        rows, k, cols, decay_factor, _ptr(decay_device), int(has_decay), cta_warps, _ptr(decay_job),
        _stream(weights[0])))


def decay_job_bytes() -> int:
    """Bytes of device memory one decay job takes."""
    return int(library().dionw_decay_job_bytes())


def decay_job_begin(job: Tensor, weights: Sequence[Tensor], rowmap: Sequence[int], rows_per_tensor: Sequence[int], *,
                    rows: int, cols: int, decay_factor: float, decay_device: Tensor | None = None,
                    rows_per_wait: int = 2) -> None:
    """Write the decay job of a round into ``job`` (a byte tensor of ``decay_job_bytes()``): the
    round's weights in the order ``apply_round`` will get them, ``rowmap[i]`` the device address of
    tensor ``i``'s int32 row map."""
    n = len(weights)
    _check(library().dionw_decay_job_begin(
        job.data_ptr(), _ptr_array(weights), (c_void_p * n)(*rowmap), _i64_array(rows_per_tensor), n, rows, cols,
        decay_factor, _ptr(decay_device), rows_per_wait, _stream(job)))


def gemm_side_job(job: Tensor | None) -> None:
    """Products launched by this thread from now on carry ``job`` (None: no job)."""
    library().dionw_gemm_side_job(_ptr(job))


def write_scalars(dst: Tensor, values: Sequence[float]) -> None:
    """``dst[:len(values)] = values`` (fp32, on the device), ordered on the current stream."""
    n = len(values)
    _check(library().dionw_write_scalars(dst.data_ptr(), (c_float * n)(*values), n, _stream(dst)))


# ---------------------------------------------------------------------------
# AdamW and EMA
# ---------------------------------------------------------------------------
def adamw_multi(params: Sequence[Tensor], grads: Sequence[Tensor], exp_avg: Sequence[Tensor],
                exp_avg_sq: Sequence[Tensor], steps: Sequence[Tensor], *, lr: float, beta1: float, beta2: float,
                weight_decay: float, eps: float, hyper_device: Tensor | None = None) -> None:
    """``hyper_device`` (two fp32 on the device: lr, weight decay) overrides the two host values."""
    if not params:
        return
    _check(library().dionw_adamw_multi(
        _ptr_array(params), _ptr_array(grads), _ptr_array(exp_avg), _ptr_array(exp_avg_sq), _ptr_array(steps),
        _i64_array([p.numel() for p in params]), len(params), lr, beta1, beta2, weight_decay, eps,
        _ptr(hyper_device), _stream(params[0])))


def ema_multi(shadows: Sequence[Tensor], sources: Sequence[Tensor], *, weight: float, first: bool) -> None:
    """Tensors of one source dtype per call."""
    if not shadows:
        return
    _check(library().dionw_ema_multi(
        _ptr_array(shadows), _ptr_array(sources), _i64_array([s.numel() for s in shadows]), len(shadows),
        dtype_code(sources[0].dtype), weight, int(first), _stream(shadows[0])))


def ema_stage_pack(sources: Sequence[Tensor], offsets: Sequence[int], staging: Tensor) -> None:
    if not sources:
        return
    _check(library().dionw_ema_stage_pack(
        _ptr_array(sources), _i64_array([s.numel() for s in sources]), _i64_array(offsets), len(sources),
        dtype_code(sources[0].dtype), staging.data_ptr(), _stream(sources[0])))


class CpuEmaJob:
    """Handle of one host-side EMA update running on the library's worker thread."""

    def __init__(self, shadows: Sequence[Tensor], staged: Sequence[Tensor], first: Sequence[bool], weight: float,
                 event: "torch.cuda.Event | None", threads: int) -> None:
        self._keep = (list(shadows), list(staged), event)
        n = len(shadows)
        flags = (c_uint8 * n)(*[1 if f else 0 for f in first])
        handle = library().dionw_cpu_ema_job_start(
            _ptr_array(shadows), _ptr_array(staged), _i64_array([s.numel() for s in shadows]), flags, n, weight,
            None if event is None else event.cuda_event, threads)
        if not handle:
            raise RuntimeError(f"dionw_b200: {last_error()}")
        self._handle = c_void_p(handle)

    def wait_copy(self) -> None:
        _check(library().dionw_cpu_ema_job_wait_copy(self._handle))

    def wait_update(self) -> None:
        _check(library().dionw_cpu_ema_job_wait_update(self._handle))

    def done(self) -> bool:
        return bool(library().dionw_cpu_ema_job_done(self._handle))

    def close(self) -> None:
        if self._handle is not None:
            library().dionw_cpu_ema_job_destroy(self._handle)
            self._handle = None

    def __del__(self) -> None:  # pragma: no cover - interpreter shutdown order
        try:
            self.close()
        except Exception:
            pass
