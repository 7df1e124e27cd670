"""The kernels of the engine, as Python functions over torch tensors.

Each function checks its arguments, then calls one ``extern "C"`` launcher of the
package's CUDA library on torch's current stream.  Outputs are written into
tensors the caller provides; nothing here allocates device memory.  There is no
CPU path: the first call loads the library (building it when needed) and raises
if that fails or if a tensor is not on a CUDA device.

Matrix products: the float32 path uses the package's own FFMA kernel
(``gemm_f32.cu``: true 32-bit, fixed summation order).  The bfloat16 path has two
kernels of its own: weight streaming for up to 8 rows (``gemm_skinny.cu``, every
decode step of up to 8 requests) and tcgen05 / TMA / TMEM for many rows
(``gemm_tcgen05.cu``, switched on with ``set_tcgen05_min_rows``).  Otherwise it calls
cuBLAS through ``torch.mm``, as cklxx/arle calls cuBLASLt for all its projections
(crates/cuda-kernels/csrc/gemm/gemv.cu:298-482).
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from . import build as _build

_LIB = None
_LAUNCHES = 0


def launch_count() -> int:
    """Kernels of this package launched so far (graph replays count what they hold)."""
    return _LAUNCHES


def add_launches(n: int) -> None:
    global _LAUNCHES
    _LAUNCHES += n


_P, _I, _F = c_void_p, c_int, c_float
_SIGNATURES = {
    "arle_embedding": [_P, _P, _I, _P, _I, _I, _I, _P, _P, _P, _P],
    "arle_rmsnorm": [_P, _P, _P, _P, _P, _I, _I, _I, _F, _I, _P],
    "arle_residual_add": [_P, _P, _I, _I, _I, _P],
    "arle_silu_mul": [_P, _P, _I, _I, _I, _P],
    "arle_attention_prep": [_P, _I, _I, _P, _P, _P, _P, _F, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P],
    "arle_rotary_angles": [_P, _P, _P, _I, _I, _P],
    "arle_paged_attention_plain": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "arle_paged_attention_decode": [_P, _I, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P],
    "arle_paged_attention_decode_stream": [_P, _I, _P, _P, _P, ctypes.c_longlong, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I,
                                           _F, _I, _I, _I, _P, _P],
    "arle_paged_attention_decode_stream_prep": [_P, _I, _P, _P, _P, ctypes.c_longlong, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I,
                                                _F, _I, _I, _I, _I, _P, _P, _P, _F, _P, _P, _P, _P],
    "arle_decode_stream_plan_ints": [_I, _I],
    "arle_decode_stream_plan": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "arle_paged_attention_prefill": [_P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _I, _P],
    "arle_paged_attention_prefill_tc": [_P, _I, _I, _P, _P, _P, ctypes.c_longlong, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I,
                                        _I, _I, _I, _P, _P],
    "arle_gemm_f32": [_P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P],
    "arle_gemm_plain_bf16": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "arle_gemm_skinny": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _P, _P],
    "arle_gemm_skinny_gated": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _P, _P],
    "arle_gemm_skinny_fused": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _F, _F, _P, _I, _P, _P, _I, _P, _P, _P],
    "arle_gemm_tcgen05": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _P, _P],
    "arle_gemm_tcgen05_pair": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "arle_argmax": [_P, _I, _I, _I, _P, _P, _P, _P, _P],
    "arle_scatter_tokens": [_P, _P, _P, _I, _P],
    "arle_sample": [_P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P],
}


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The loaded CUDA library; built on first use.  Raises if it cannot be had."""
    global _LIB
    if _LIB is None:
        path = _build.library_path()
        lib = ctypes.CDLL(path)
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = c_int
        _LIB = lib
    return _LIB


_ERR_FLAGS = {}


def _device_key(device) -> torch.device:
    """"cuda" and "cuda:0" name the same device: always the indexed form."""
    d = torch.device(device)
    if d.type == "cuda" and d.index is None:
        d = torch.device("cuda", torch.cuda.current_device())
    return d


def error_flag(device) -> torch.Tensor:
    """The device word that kernels with bounded waits raise when a wait ran out
    (one int32 per device, made at first use)."""
    key = _device_key(device)
    if key not in _ERR_FLAGS:
        _ERR_FLAGS[key] = torch.zeros(1, dtype=torch.int32, device=key)
    return _ERR_FLAGS[key]


def check_errors(device) -> None:
    """Reads the error word (a device synchronisation) and raises if a kernel gave
    up waiting; the word is cleared."""
    key = _device_key(device)
    if key in _ERR_FLAGS:
        code = int(_ERR_FLAGS[key].item())
        if code != 0:
            _ERR_FLAGS[key].zero_()
            raise KernelError(f"a kernel gave up a bounded wait (code {code}: an asynchronous copy or a tensor-core "
                              "operation did not complete); results are invalid")


def set_programmatic_launch(on) -> None:
    """Programmatic dependent launch (off by default): a kernel may be scheduled, set up
    its barriers and prefetch weights while the kernel before it finishes, and waits
    for that kernel only before touching its results.  True or 1: every kernel; 2: the
    weight-streaming products only."""
    lib = library()
    lib.arle_set_programmatic_launch.argtypes = [c_int]
    lib.arle_set_programmatic_launch.restype = None
    lib.arle_set_programmatic_launch(int(on))


_KERNEL_SET = "fast"


class use_kernel_set:
    """``with use_kernel_set("plain"):`` makes every dispatch inside it take the general
    kernels (plain FFMA products with float32 sums, the general paged attention, the gate
    as a kernel of its own), whatever the shapes; "fast" (the default) lets the shapes
    decide.  The plain set is the yardstick a bfloat16 discrepancy is bisected with:
    the same trace on both sets differs only by the fast kernels.  cklxx/arle chooses a
    backend per operation in the same place (infer/src/ops.rs:135-269)."""

    def __init__(self, name: str):
        if name not in ("fast", "plain"):
            raise ValueError(f"kernel set must be 'fast' or 'plain', got {name!r}")
        self.name = name

    def __enter__(self):
        global _KERNEL_SET
        self._before = _KERNEL_SET
        _KERNEL_SET = self.name
        return self

    def __exit__(self, *exc):
        global _KERNEL_SET
        _KERNEL_SET = self._before
        return False


def kernel_set() -> str:
    return _KERNEL_SET


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported dtype {t.dtype}: the kernels take float32 and bfloat16")


def _ptr(t, name="tensor"):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}: arle_b200 kernels run on CUDA devices only (there is no CPU path)")
    return t.data_ptr()


def _stream():
    # torch's raw-stream query: a plain C call (torch.cuda.current_stream() builds a Python object and costs
    # some 15 us, once per launch)
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


def _check(code: int, what: str):
    global _LAUNCHES
    if code == 0:
        _LAUNCHES += 1
        return
    if code == -2:
        raise KernelError(f"{what}: sizes not supported by this kernel")
    if code == -3:
        raise KernelError(f"{what}: bad argument")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _i32(t, name):
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")
    return t


# ------------------------------------------------------------------- embedding
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor = None,
              last_token: torch.Tensor = None, slot_of_token: torch.Tensor = None) -> None:
    """out[t, :] = float32(table[ids[t], :]).  ids int32 [T]; out float32 [T, H].  With
    ``last_token`` (int32, one entry per request slot) and ``slot_of_token`` (int32 [T]) a
    negative id stands for last_token[slot_of_token[t]], the token the request sampled last."""
    T, H = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embedding: out must be contiguous float32 and the table contiguous")
    if ids.numel() != T or table.shape[1] != H:
        raise KernelError(f"embedding: shapes ids {tuple(ids.shape)} table {tuple(table.shape)} out {tuple(out.shape)}")
    _i32(ids, "ids")
    if last_token is not None:
        _i32(last_token, "last_token"), _i32(slot_of_token, "slot_of_token")
        if slot_of_token is None or slot_of_token.numel() != T:
            raise KernelError("embedding: slot_of_token must name a slot for every token")
    _check(library().arle_embedding(_ptr(ids), _ptr(table), _dt(table), _ptr(out), T, H, table.shape[0],
                                    _ptr(err), _ptr(last_token), _ptr(slot_of_token) if last_token is not None else None,
                                    _stream()), "embedding")


# ------------------------------------------------------------------------ norm
def rmsnorm(resid, delta, rows, weight, eps: float, out, write_resid: bool) -> None:
    """For output row i (source row r = rows[i], or i): x = resid[r] (+ delta[r]);
    resid[r] = x when write_resid; out[i] = x * rsqrt(mean(x^2) + eps) * weight.
    resid float32 [N, H]; delta and out in the activation type; weight float32 [H]."""
    H = resid.shape[1]
    n_out = out.shape[0]
    if resid.dtype != torch.float32 or weight.dtype != torch.float32:
        raise KernelError("rmsnorm: residual and weight must be float32")
    if not (resid.is_contiguous() and out.is_contiguous()) or out.shape[1] != H or weight.numel() != H:
        raise KernelError("rmsnorm: bad shapes or strides")
    if delta is not None and (delta.dtype != out.dtype or delta.shape != resid.shape or not delta.is_contiguous()):
        raise KernelError("rmsnorm: delta must match the residual's shape and the output's type")
    if rows is not None:
        _i32(rows, "rows")
        if rows.numel() != n_out:
            raise KernelError("rmsnorm: one output row per entry of rows")
    elif n_out != resid.shape[0]:
        raise KernelError("rmsnorm: output rows must match residual rows when no row list is given")
    _check(library().arle_rmsnorm(_ptr(resid), _ptr(delta), _ptr(rows), _ptr(weight), _ptr(out), _dt(out), n_out, H,
                                  float(eps), int(bool(write_resid)), _stream()), "rmsnorm")


def residual_add(resid, delta) -> None:
    """resid += delta (float32 residual, delta in the activation type)."""
    if resid.dtype != torch.float32 or resid.shape != delta.shape or not (resid.is_contiguous() and delta.is_contiguous()):
        raise KernelError("residual_add: residual float32, same contiguous shape as delta")
    _check(library().arle_residual_add(_ptr(resid), _ptr(delta), _dt(delta), resid.shape[0], resid.shape[1], _stream()),
           "residual_add")


# ------------------------------------------------------------------------ gemm
SS_TABLE_SHAPE = (16, 192)          # a sum-of-squares table of the fused products: [rows, slots], float32


class ResidualSink:
    """Where a product's result goes instead of an output tensor, so that the norm that follows
    needs no kernel: the sums are added into ``resid`` (float32 [M, N], in place), ``xs`` gets
    bfloat16(resid * gamma) (the norm's output without its per-row factor) and ``ss`` (float32
    ``SS_TABLE_SHAPE``) the sums of squares of the new residual rows, spread over slots that the
    reader adds up.  ``eps`` travels with it to the reader."""

    def __init__(self, resid, gamma, eps, xs, ss):
        self.resid, self.gamma, self.eps, self.xs, self.ss = resid, gamma, float(eps), xs, ss
        self.filled = False


class ScaledRows:
    """Rows that still lack the per-row factor of their RMSNorm: the normalised rows are
    ``rows[m] * rsqrt(sum(ss[m, :]) / rows.shape[1] + eps)``.  A product over such rows applies
    the factor to its sums (``gemm(..., row_scale=...)``)."""

    def __init__(self, rows, ss, eps):
        self.rows, self.ss, self.eps = rows, ss, float(eps)

    @property
    def shape(self):
        return self.rows.shape

    @property
    def dtype(self):
        return self.rows.dtype


def fused_gemm_supported(x, w) -> bool:
    """The fusions live in the weight-streaming kernel: bfloat16, up to 8 rows, its alignment rules,
    and the fast kernel set."""
    return (_KERNEL_SET == "fast" and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.shape[0] <= 8 and x.shape[1] % 32 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def fused_gemm_shape_ok(rows: int, w: torch.Tensor, gated: bool = False) -> bool:
    """Whether a product of ``rows`` bfloat16 rows with ``w`` can take the fused kernel (asked by the
    parts before they hand out a sink or rows without their norm factor)."""
    return (_KERNEL_SET == "fast" and w is not None and w.is_cuda and w.dtype == torch.bfloat16 and 0 < rows <= 8
            and w.shape[1] % 32 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0
            and (not gated or gated_gemm_fits(w.shape[1])))


def _fused_gemm(x, w, out, gated: bool, scaled: "ScaledRows", sink: "ResidualSink") -> None:
    M, K = x.shape
    N = w.shape[0]
    in_ss = inv_w = eps = None
    if scaled is not None:
        if scaled.ss.dtype != torch.float32 or tuple(scaled.ss.shape) != SS_TABLE_SHAPE or not scaled.ss.is_contiguous():
            raise KernelError("gemm: a row-scale table must be contiguous float32 of SS_TABLE_SHAPE")
        in_ss, inv_w, eps = scaled.ss, 1.0 / K, scaled.eps
    if sink is not None:
        r, xs = sink.resid, sink.xs
        if (r.dtype != torch.float32 or tuple(r.shape) != (M, N) or r.stride(1) != 1 or xs.dtype != torch.bfloat16
                or tuple(xs.shape) != (M, N) or xs.stride(1) != 1 or sink.gamma.dtype != torch.float32
                or sink.gamma.numel() != N or tuple(sink.ss.shape) != SS_TABLE_SHAPE or sink.ss.dtype != torch.float32):
            raise KernelError("gemm: residual sink does not fit the product")
    _check(library().arle_gemm_skinny_fused(
        _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), _dt(out) if out is not None else 1,
        out.stride(0) if out is not None else 0, M, N, K, int(gated), _ptr(in_ss), float(inv_w or 0.0), float(eps or 0.0),
        _ptr(sink.resid) if sink else None, sink.resid.stride(0) if sink else 0, _ptr(sink.gamma) if sink else None,
        _ptr(sink.xs) if sink else None, sink.xs.stride(0) if sink else 0, _ptr(sink.ss) if sink else None,
        _ptr(error_flag(x.device)), _stream()), "gemm_skinny_fused")
    if sink is not None:
        sink.filled = True


def gemm(x, w: torch.Tensor, out: torch.Tensor, sink: "ResidualSink" = None) -> bool:
    """out[M, N] = x[M, K] . w[N, K]^T (weights stored [out_features, in_features]).

    ``x`` may be ``ScaledRows`` (the product then applies their per-row factor).  With a ``sink`` the
    result is added into the residual instead (see ``ResidualSink``) when the shapes allow the fused
    kernel; the return value says whether that happened (if not, ``out`` holds the product as
    usual and the sink is untouched)."""
    scaled = x if isinstance(x, ScaledRows) else None
    if scaled is not None:
        x = scaled.rows
    if scaled is not None or sink is not None:
        if fused_gemm_supported(x, w) and w.shape[1] == x.shape[1]:
            use_sink = sink is not None
            _fused_gemm(x, w, None if use_sink else out, False, scaled, sink)
            return use_sink
        if scaled is not None:
            raise KernelError("gemm: rows that lack their norm factor need the fused weight-streaming kernel "
                              f"(bfloat16, up to 8 rows, K a multiple of 32); got x {tuple(x.shape)} {x.dtype}")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm: shapes x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    if x.dtype == torch.float32:
        if out.dtype != torch.float32 or x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("gemm: the float32 path takes float32 activations with unit inner stride")
        _check(library().arle_gemm_f32(_ptr(x), _ptr(w), _dt(w), _ptr(out), M, N, K, x.stride(0), w.stride(0),
                                       out.stride(0), _stream()), "gemm_f32")
        return False
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm: bfloat16 path needs bfloat16 operands, got {x.dtype} and {w.dtype}")
    _ptr(x), _ptr(w), _ptr(out)
    if _KERNEL_SET == "plain":
        if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("gemm: operands need unit inner strides")
        _check(library().arle_gemm_plain_bf16(_ptr(x), _ptr(w), _ptr(out), _dt(out), M, N, K, x.stride(0), w.stride(0),
                                              out.stride(0), _stream()), "gemm_plain_bf16")
        return False
    if skinny_gemm_supported(x, w, out):
        _check(library().arle_gemm_skinny(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), _dt(out), out.stride(0),
                                          M, N, K, _ptr(error_flag(x.device)), _stream()), "gemm_skinny")
        return False
    if M >= _TCGEN05_MIN_ROWS and tcgen05_gemm_supported(x, w, out):
        gemm_tcgen05(x, w, out)
        return False
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    elif out.dtype == torch.float32:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    else:
        raise KernelError(f"gemm: output type {out.dtype}")
    return False


_TCGEN05_MIN_ROWS = 1 << 30


def set_tcgen05_min_rows(rows: int) -> None:
    """bfloat16 products with at least this many rows of x run on the package's tcgen05
    kernel instead of cuBLAS.  Off by default (a very large value): the kernel reaches
    85 to 90 % of cuBLAS at 2,048 rows and falls behind it below 512, so cuBLAS stands
    for these products, as cuBLASLt does in cklxx/arle."""
    global _TCGEN05_MIN_ROWS
    _TCGEN05_MIN_ROWS = int(rows)


def tcgen05_gemm_supported(x, w, out) -> bool:
    """The tcgen05 kernel takes bfloat16 operands with K and the row strides multiples
    of 8 elements and 16-byte aligned bases (what its TMA tensor maps need)."""
    K = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(1) == 1
            and w.stride(1) == 1 and out.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.dtype in (torch.bfloat16, torch.float32))


def gemm_tcgen05(x, w, out) -> None:
    """out[M, N] = x[M, K] . w[N, K]^T on the tcgen05 tensor cores (TMA-fed, TMEM accumulators)."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N or not tcgen05_gemm_supported(x, w, out):
        raise KernelError(f"gemm_tcgen05: unsupported operands x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    _check(library().arle_gemm_tcgen05(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), _dt(out), out.stride(0), M, N,
                                       K, _ptr(error_flag(x.device)), _stream()), "gemm_tcgen05")


def gemm_tcgen05_pair(x, w, out, gated: bool = False) -> None:
    """out[M, N] = x[M, K] . w[N, K]^T on the tcgen05 tensor cores with two SMs to a 256 x 256 tile
    (``cta_group::2``).  ``gated``: w holds (gate_i, up_i) in rows 2i and 2i + 1 and out [M, N / 2] gets
    silu(gate) * up, the gate applied to the float32 sums in the kernel's epilogue."""
    M, K = x.shape
    N = w.shape[0]
    No = N // 2 if gated else N
    if (w.shape[1] != K or out.shape[0] != M or out.shape[1] != No or not tcgen05_gemm_supported(x, w, out)
            or (gated and (N % 2 or out.dtype != torch.bfloat16))):
        raise KernelError(f"gemm_tcgen05_pair: unsupported operands x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    _check(library().arle_gemm_tcgen05_pair(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), _dt(out), out.stride(0), M,
                                            N, K, int(bool(gated)), _ptr(error_flag(x.device)), _stream()),
           "gemm_tcgen05_pair")


def skinny_gemm_supported(x, w, out) -> bool:
    """The weight-streaming kernel takes up to 8 rows of x (the kernel itself up to 16, where cuBLAS is faster), K a multiple of 32, rows
    that start on 16-byte boundaries and unit inner strides."""
    M, K = x.shape
    return (M <= 8 and K % 32 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and out.dtype in (torch.bfloat16, torch.float32))


# ------------------------------------------------------------------- attention
def rotary_angles(positions, inv_freq, out) -> None:
    """out[t, i] = (cos, sin)(positions[t] * inv_freq[i]) in float32, [T, len(inv_freq), 2]: what
    ``attention_prep`` evaluates for every layer of a step, once."""
    T, half = positions.numel(), inv_freq.numel()
    if (out.dtype != torch.float32 or tuple(out.shape) != (T, half, 2) or not out.is_contiguous()
            or inv_freq.dtype != torch.float32):
        raise KernelError("rotary_angles: out must be contiguous float32 [T, len(inv_freq), 2]")
    _i32(positions, "positions")
    _check(library().arle_rotary_angles(_ptr(positions), _ptr(inv_freq), _ptr(out), T, half, _stream()), "rotary_angles")


def attention_prep_takes_angles(qkv, hd: int, rotary_dim: int) -> bool:
    """Whether ``attention_prep`` would use a table of ``rotary_angles`` for this input (the kernel for
    prompt portions does; the others evaluate the angles themselves)."""
    return qkv.dtype == torch.bfloat16 and qkv.shape[0] >= 32 and hd in (64, 128) and rotary_dim == hd


def attention_prep(qkv, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, rotary_dim, k_cache, v_cache,
                   nq: int, nkv: int, hd: int, page_size: int, angles=None) -> None:
    """Per-head q/k RMSNorm (weights float32 [hd] or None), rotary encoding, and the
    store of k and v into the paged cache, in place on qkv [T, (nq + 2 nkv) hd]
    (nkv = 0: the rows hold q only and nothing is stored).  ``angles``: the table of
    ``rotary_angles`` for these positions and inv_freq, or None."""
    T = qkv.shape[0]
    if angles is not None and (angles.dtype != torch.float32 or tuple(angles.shape) != (T, rotary_dim // 2, 2)
                               or not angles.is_contiguous()):
        raise KernelError("attention_prep: angles must be contiguous float32 [T, rotary_dim / 2, 2]")
    if qkv.stride(1) != 1 or qkv.shape[1] < (nq + 2 * nkv) * hd:
        raise KernelError("attention_prep: qkv must be [T, >= (nq + 2 nkv) hd] with unit inner stride")
    if hd % 2 or hd > 256:
        raise KernelError(f"attention_prep: head_dim {hd} not supported (even, at most 256)")
    for w_ in (q_weight, k_weight):
        if w_ is not None and (w_.dtype != torch.float32 or w_.numel() != hd):
            raise KernelError("attention_prep: norm weights must be float32 [head_dim]")
    if nkv > 0:
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
            raise KernelError("attention_prep: cache type differs from activation type")
        if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or k_cache.shape != v_cache.shape:
            raise KernelError(f"attention_prep: cache shape {tuple(k_cache.shape)} is not [pages, {nkv}, {page_size}, {hd}]")
        if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
            raise KernelError("attention_prep: cache layers must be contiguous")
        _i32(slot_mapping, "slot_mapping")
    _i32(positions, "positions")
    if rotary_dim and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("attention_prep: inv_freq must be float32 [rotary_dim / 2]")
    _check(library().arle_attention_prep(
        _ptr(qkv), _dt(qkv), qkv.stride(0), _ptr(positions), _ptr(slot_mapping), _ptr(q_weight), _ptr(k_weight),
        float(eps), _ptr(inv_freq) if rotary_dim else None, _ptr(angles) if rotary_dim else None, int(rotary_dim),
        _ptr(k_cache) if nkv else None,
        _ptr(v_cache) if nkv else None, nq, nkv, hd, page_size, T, _stream()), "attention_prep")


def paged_attention(q, out, k_cache, v_cache, positions, row_of_token, block_table, nq: int, nkv: int, hd: int,
                    page_size: int, scale: float, window, batch=None) -> None:
    """Causal attention of this step's queries over the paged cache.

    q: [T, nq*hd] view (row stride free, unit inner stride); out: contiguous
    [T, nq*hd]; caches [pages, nkv, page_size, hd]; positions / row_of_token int32
    [T]; block_table int32 [rows, max_pages].  ``window`` None or <= 0 means all
    keys.  ``batch`` (a StepContext) lets faster kernels pick their launch shape;
    the general kernel does not need it."""
    T = q.shape[0]
    if q.stride(1) != 1 or q.shape[1] != nq * hd or out.shape != (T, nq * hd) or not out.is_contiguous():
        raise KernelError("paged_attention: q must be [T, nq*hd] with unit inner stride and out contiguous [T, nq*hd]")
    if q.dtype != k_cache.dtype or out.dtype != q.dtype:
        raise KernelError("paged_attention: q, out and cache must share a type")
    if hd > 256 or nq % nkv:
        raise KernelError(f"paged_attention: head_dim {hd} / heads {nq}:{nkv} not supported")
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError(f"paged_attention: cache shape {tuple(k_cache.shape)} is not [pages, {nkv}, {page_size}, {hd}]")
    _i32(positions, "positions"), _i32(row_of_token, "row_of_token"), _i32(block_table, "block_table")
    if block_table.stride(1) != 1:
        raise KernelError("paged_attention: block table rows must be contiguous")
    if batch is not None and _KERNEL_SET == "fast" and fast_attention_supported(q, nq, nkv, hd):
        if batch.max_q_len > 1:
            prefill = paged_attention_prefill_tc if tc_attention_supported(q, hd, page_size) else paged_attention_prefill
            prefill(q, out, k_cache, v_cache, batch.q_indptr, batch.kv_lens, block_table, nq, nkv, hd, page_size, scale,
                    window, batch.max_q_len, skip_single=batch.num_single > 0)
        if batch.num_single > 0 and stream_decode_supported(batch.num_rows, page_size, nq // nkv):
            ctas = sm_count(q.device)
            slots = (ctas + batch.num_rows * nkv) * (nq // nkv)
            paged_attention_decode_stream(
                q, out, k_cache, v_cache, batch.q_indptr, batch.kv_lens, block_table, nq, nkv, hd, page_size, scale, window,
                batch.ws.get("attn_piece_o", (slots * hd,), torch.float32),
                batch.ws.get("attn_piece_ml", (slots * 2,), torch.float32),
                batch.ws.get_zeroed("attn_piece_counters", (batch.num_rows * nkv,), torch.int32), ctas)
        elif batch.num_single > 0:
            splits = decode_splits(batch.num_rows, nkv, block_table.shape[1] * page_size, q.device)
            part_o = part_ml = counters = None
            if splits > 1:
                part_o = batch.ws.get("attn_part_o", (batch.num_rows * nq * splits * hd,), torch.float32)
                part_ml = batch.ws.get("attn_part_ml", (batch.num_rows * nq * splits * 2,), torch.float32)
                counters = batch.ws.get_zeroed("attn_split_counters", (batch.num_rows * nkv,), torch.int32)
            paged_attention_decode(q, out, k_cache, v_cache, batch.q_indptr, batch.kv_lens, block_table, nq, nkv, hd,
                                   page_size, scale, window, splits, part_o, part_ml, counters)
        return
    _check(library().arle_paged_attention_plain(
        _ptr(q), q.stride(0), _ptr(out), _ptr(k_cache), _ptr(v_cache), _dt(q), _ptr(positions), _ptr(row_of_token),
        _ptr(block_table), block_table.stride(0), nq, nkv, hd, page_size, float(scale),
        int(window) if window else 0, T, _stream()), "paged_attention")


def fast_attention_supported(q, nq: int, nkv: int, hd: int) -> bool:
    """The tensor-core attention kernels take bfloat16, head sizes 64 and 128, up to
    16 query heads per kv head and 16-byte aligned query rows; everything else
    runs on the general kernel."""
    return (q.dtype == torch.bfloat16 and hd in (64, 128) and nq // nkv <= 16 and q.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0)


def tc_attention_supported(q, hd: int, page_size: int) -> bool:
    """The tcgen05 prefill kernel takes head size 128 and pages of a multiple of 16 tokens."""
    return hd == 128 and page_size % 16 == 0 and q.dtype == torch.bfloat16


def paged_attention_prefill_tc(q, out, k_cache, v_cache, q_indptr, kv_lens, block_table, nq, nkv, hd, page_size, scale,
                               window, max_q_len: int, skip_single: bool = False) -> None:
    """Flash attention over the paged cache on the tcgen05 tensor cores (TMA-fed, scores
    and output in tensor memory) for rows with several queries."""
    R = kv_lens.numel()
    _i32(q_indptr, "q_indptr"), _i32(kv_lens, "kv_lens"), _i32(block_table, "block_table")
    if not tc_attention_supported(q, hd, page_size) or q.stride(1) != 1 or not out.is_contiguous():
        raise KernelError("paged_attention_prefill_tc: needs bfloat16, head size 128, page size a multiple of 16")
    _check(library().arle_paged_attention_prefill_tc(
        _ptr(q), q.stride(0), q.shape[0], _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(q_indptr),
        _ptr(kv_lens), _ptr(block_table), block_table.stride(0), block_table.shape[1], nq, nkv, hd, page_size, float(scale),
        int(window) if window else 0, R, int(max_q_len), int(bool(skip_single)), _ptr(error_flag(q.device)), _stream()),
        "paged_attention_prefill_tc")


_SM_COUNT: dict = {}


def sm_count(device=None) -> int:
    device = torch.device(device if device is not None else "cuda")
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _SM_COUNT[key]


def stream_decode_supported(rows: int, page_size: int, group: int = 1) -> bool:
    """The streaming decode kernel fetches keys in TMA boxes of 16: pages must be
    multiples of 16; its row table lives in shared memory: up to 2,048 rows; the query
    heads of a kv head are the 16 rows of one MMA."""
    return page_size % 16 == 0 and rows <= 2048 and group <= 16


def paged_attention_decode_stream(q, out, k_cache, v_cache, q_indptr, kv_lens, block_table, nq, nkv, hd, page_size, scale,
                                  window, piece_o, piece_ml, counters, ctas: int) -> None:
    """Attention of the rows that have exactly one query (others are skipped), as a
    resident grid of ``ctas`` CTAs that share the batch's 64-key tiles evenly.
    Scratch: piece_o float32 [(ctas + R*nkv) * (nq/nkv) * hd], piece_ml float32
    [(ctas + R*nkv) * (nq/nkv) * 2], counters int32 [R*nkv], zero before the first
    launch (the kernel leaves it zero)."""
    R = kv_lens.numel()
    slots = (ctas + R * nkv) * (nq // nkv)
    if (piece_o.numel() < slots * hd or piece_ml.numel() < slots * 2 or counters.numel() < R * nkv
            or piece_o.dtype != torch.float32 or piece_ml.dtype != torch.float32 or counters.dtype != torch.int32):
        raise KernelError("paged_attention_decode_stream: scratch for the pieces is missing or too small")
    if q.dtype != torch.bfloat16 or q.stride(1) != 1 or not out.is_contiguous():
        raise KernelError("paged_attention_decode_stream: needs bfloat16 queries with unit inner stride")
    if not stream_decode_supported(R, page_size, nq // nkv):
        raise KernelError(f"paged_attention_decode_stream: {R} rows with {nq // nkv} query heads per kv head and pages of "
                          f"{page_size} are outside what this kernel takes")
    _i32(q_indptr, "q_indptr"), _i32(kv_lens, "kv_lens"), _i32(block_table, "block_table")
    _check(library().arle_paged_attention_decode_stream(
        _ptr(q), q.stride(0), _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(q_indptr), _ptr(kv_lens),
        _ptr(block_table), block_table.stride(0), block_table.shape[1], _ptr(piece_o), _ptr(piece_ml), _ptr(counters),
        nq, nkv, hd, page_size, float(scale), int(window) if window else 0, R, int(ctas), _ptr(error_flag(q.device)),
        _stream()), "paged_attention_decode_stream")


def fused_decode_supported(qkv, batch, cache_dtype, nq: int, nkv: int, hd: int, page_size: int, rotary_dim: int) -> bool:
    """Whether a step's attention can run as ONE launch that also prepares the queries and the new keys
    (``decode_attention_with_prep``): every row of the step one decoded token, bfloat16, the shapes the
    streaming kernel takes, and a rotation of the whole head or none."""
    return (_KERNEL_SET == "fast" and batch is not None and batch.max_q_len == 1 and qkv.is_cuda
            and qkv.dtype == torch.bfloat16 and cache_dtype == torch.bfloat16 and hd in (64, 128) and nq % nkv == 0
            and nq // nkv <= 16 and rotary_dim in (0, hd) and stream_decode_supported(batch.num_rows, page_size, nq // nkv)
            and qkv.stride(1) == 1 and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0)


def decode_attention_with_prep(qkv, out, k_cache, v_cache, slot_mapping, q_weight, k_weight, eps: float, inv_freq,
                               block_table, nq: int, nkv: int, hd: int, page_size: int, scale: float, window, batch) -> None:
    """Attention of a step in which every row is one decoded token, from the raw projection output
    qkv [T, (nq + 2 nkv) hd]: per-head norm and rotation of the queries and of the new keys, the store of
    the new keys and values into the cache, and the attention over the cache, in one launch of the
    streaming kernel.  ``q_weight`` / ``k_weight`` None: no norm; ``inv_freq`` None: no rotation."""
    T = qkv.shape[0]
    if not fused_decode_supported(qkv, batch, k_cache.dtype, nq, nkv, hd, page_size, hd if inv_freq is not None else 0):
        raise KernelError("decode_attention_with_prep: this step or these shapes need the separate preparation kernel")
    if out.shape != (T, nq * hd) or not out.is_contiguous() or out.dtype != torch.bfloat16 or qkv.shape[1] < (nq + 2 * nkv) * hd:
        raise KernelError("decode_attention_with_prep: out must be contiguous bfloat16 [T, nq*hd] and qkv hold q, k and v heads")
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or k_cache.shape != v_cache.shape or not (
            k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelError(f"decode_attention_with_prep: cache shape {tuple(k_cache.shape)} is not [pages, {nkv}, {page_size}, {hd}]")
    for w_ in (q_weight, k_weight):
        if w_ is not None and (w_.dtype != torch.float32 or w_.numel() != hd):
            raise KernelError("decode_attention_with_prep: norm weights must be float32 [head_dim]")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != hd // 2):
        raise KernelError("decode_attention_with_prep: inv_freq must be float32 [head_dim / 2]")
    _i32(slot_mapping, "slot_mapping"), _i32(block_table, "block_table")
    R, G = batch.num_rows, nq // nkv
    ctas = sm_count(qkv.device)
    slots = (ctas + R * nkv) * G
    piece_o = batch.ws.get("attn_piece_o", (slots * hd,), torch.float32)
    piece_ml = batch.ws.get("attn_piece_ml", (slots * 2,), torch.float32)
    counters = batch.ws.get_zeroed("attn_piece_counters", (R * nkv,), torch.int32)
    # How the keys are shared out among the CTAs, and which pages each CTA reads first, depends on the rows' lengths,
    # the kv heads, the window and the group's block table alone: worked out by the step's first layer for all that
    # follow (the step's memo, where there is one)
    plan = None
    memo = getattr(batch, "memo", None)
    if memo is not None:
        key = ("decode_stream_plan", nkv, int(window) if window else 0, ctas, block_table.data_ptr(), block_table.stride(0),
               block_table.shape[1], page_size)
        plan = memo.get(key)
        if plan is None:
            n = library().arle_decode_stream_plan_ints(R, int(ctas))
            plan = batch.ws.get(f"decode_stream_plan_{len(memo)}", (n,), torch.int32)
            _check(library().arle_decode_stream_plan(_ptr(batch.q_indptr), _ptr(batch.kv_lens), _ptr(block_table),
                                                     block_table.stride(0), block_table.shape[1], page_size, R, nkv, key[2],
                                                     int(ctas), _ptr(plan), _stream()), "decode_stream_plan")
            memo[key] = plan
    _check(library().arle_paged_attention_decode_stream_prep(
        _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(batch.q_indptr),
        _ptr(batch.kv_lens), _ptr(block_table), block_table.stride(0), block_table.shape[1], _ptr(piece_o), _ptr(piece_ml),
        _ptr(counters), nq, nkv, hd, page_size, float(scale), int(window) if window else 0, R, int(ctas), 1,
        _ptr(slot_mapping), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(inv_freq), _ptr(plan),
        _ptr(error_flag(qkv.device)), _stream()), "decode_attention_with_prep")


def decode_splits(rows: int, nkv: int, kv_bound: int, device=None) -> int:
    """Splits along the keys.  With enough work for four waves of CTAs (three CTAs
    per SM), one split per 512 keys; otherwise as many splits as fill one wave.
    Never more than one per 64-key tile of the longest request the tables allow."""
    slots = sm_count(device) * 3
    base = max(1, rows * nkv)
    by_len = -(-kv_bound // 512)
    splits = by_len if base * by_len >= 4 * slots else max(1, slots // base)
    return max(1, min(splits, -(-kv_bound // 64), 64))


def paged_attention_decode(q, out, k_cache, v_cache, q_indptr, kv_lens, block_table, nq, nkv, hd, page_size, scale,
                           window, splits: int, part_o=None, part_ml=None, counters=None) -> None:
    """Split-KV attention of the rows that have exactly one query (others are
    skipped).  q_indptr int32 [R+1], kv_lens int32 [R] (keys after this step).
    When splits > 1: part_o / part_ml are float32 scratch of R*nq*splits*hd and
    R*nq*splits*2 elements, counters int32 [R*nkv] that is zero before the first
    launch (the kernel leaves it zero)."""
    R = kv_lens.numel()
    if splits > 1 and (part_o is None or part_ml is None or counters is None or part_o.numel() < R * nq * splits * hd
                       or part_ml.numel() < R * nq * splits * 2 or part_o.dtype != torch.float32
                       or counters.dtype != torch.int32 or counters.numel() < R * nkv):
        raise KernelError("paged_attention_decode: scratch for the splits is missing or too small")
    _i32(q_indptr, "q_indptr"), _i32(kv_lens, "kv_lens"), _i32(block_table, "block_table")
    _check(library().arle_paged_attention_decode(
        _ptr(q), q.stride(0), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(q_indptr), _ptr(kv_lens),
        _ptr(block_table), block_table.stride(0), _ptr(part_o), _ptr(part_ml), _ptr(counters), nq, nkv, hd, page_size,
        float(scale), int(window) if window else 0, R, int(splits), _stream()), "paged_attention_decode")


def paged_attention_prefill(q, out, k_cache, v_cache, q_indptr, kv_lens, block_table, nq, nkv, hd, page_size, scale,
                            window, max_q_len: int, skip_single: bool = False) -> None:
    """Flash-attention over the paged cache for rows with several queries (and,
    unless skip_single, for single-query rows too)."""
    R = kv_lens.numel()
    _i32(q_indptr, "q_indptr"), _i32(kv_lens, "kv_lens"), _i32(block_table, "block_table")
    _check(library().arle_paged_attention_prefill(
        _ptr(q), q.stride(0), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(q_indptr), _ptr(kv_lens),
        _ptr(block_table), block_table.stride(0), nq, nkv, hd, page_size, float(scale),
        int(window) if window else 0, R, int(max_q_len), int(bool(skip_single)), _stream()), "paged_attention_prefill")


# ------------------------------------------------------------------ activation
def gemm_silu_mul(x: torch.Tensor, w: torch.Tensor, gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """The first half of a gated feed-forward: out[t, i] = silu(x[t] . w[2i]) * (x[t] . w[2i + 1]) for
    w [2I, K] whose rows 2i and 2i + 1 are gate_i and up_i.  Few rows of x take one launch of
    the weight-streaming kernel (the gate applied to its float32 sums); otherwise the product
    goes to ``gate_up`` [T, 2I] and ``silu_mul`` follows."""
    T, I = out.shape
    if w.shape[0] != 2 * I or gate_up.shape != (T, 2 * I):
        raise KernelError(f"gemm_silu_mul: shapes w {tuple(w.shape)} gate_up {tuple(gate_up.shape)} out {tuple(out.shape)}")
    if isinstance(x, ScaledRows):
        if not (fused_gemm_supported(x.rows, w) and gated_gemm_fits(x.rows.shape[1]) and out.stride(1) == 1):
            raise KernelError("gemm_silu_mul: rows that lack their norm factor need the gated weight-streaming kernel")
        _fused_gemm(x.rows, w, out, True, x, None)
        return
    if (_KERNEL_SET == "fast" and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and skinny_gemm_supported(x, w, out) and gated_gemm_fits(x.shape[1])):
        _ptr(x), _ptr(w), _ptr(out)
        _check(library().arle_gemm_skinny_gated(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), _dt(out), out.stride(0),
                                                T, 2 * I, x.shape[1], _ptr(error_flag(x.device)), _stream()),
               "gemm_skinny_gated")
        return
    if (_KERNEL_SET == "fast" and T >= _GATED_TCGEN05_MIN_ROWS and x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and tcgen05_gemm_supported(x, w, out)):
        gemm_tcgen05_pair(x, w, out, gated=True)
        return
    gemm(x, w, gate_up)
    silu_mul(gate_up, out)


_GATED_TCGEN05_MIN_ROWS = 1024


def set_gated_tcgen05_min_rows(rows: int) -> None:
    """Gated products (the first half of the feed-forward) with at least this many rows run on the package's
    two-SM tcgen05 kernel, which applies the gate in its epilogue, instead of cuBLAS followed by the gate
    kernel.  Default 1,024: from there on the fused kernel is at least as fast as the two together (measured
    at Qwen3-8B sizes: 293 against 300 us at 2,048 rows; at 512 rows 88 against 86)."""
    global _GATED_TCGEN05_MIN_ROWS
    _GATED_TCGEN05_MIN_ROWS = int(rows)


def gated_gemm_fits(K: int) -> bool:
    """The gate needs whole sums in one CTA: 8 rows of x (K + 8 elements each) must fit in
    shared memory beside the kernel's ring of four 32 KB stages, its reduction scratch and
    the staged table of row factors (about 147 KB of the 227 KB): K up to about 5,300."""
    return 16 * (K + 8) <= 85600


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, 2i]) * gate_up[t, 2i + 1]; gate_up [T, 2I], out [T, I]."""
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or not gate_up.is_contiguous() or not out.is_contiguous() or gate_up.dtype != out.dtype:
        raise KernelError("silu_mul: gate_up must be contiguous [T, 2I] and out contiguous [T, I] of one type")
    _check(library().arle_silu_mul(_ptr(gate_up), _ptr(out), _dt(out), T, I, _stream()), "silu_mul")


# -------------------------------------------------------------------- sampling
def argmax(logits, scratch, out, scatter=None, last_token=None) -> None:
    """out[r] = index of the largest logit of row r (ties: the lowest index), float32
    logits [R, V]; scratch float32 [R * 64].  With ``scatter`` (int32 [R]) and ``last_token``
    the token also goes to last_token[scatter[r]] (see ``embedding``)."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32 or out.numel() < R:
        raise KernelError("argmax: float32 logits with unit inner stride, int32 out with one entry per row")
    if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < R * 64:
        raise KernelError("argmax: scratch must be float32 with 64 entries per row")
    if (scatter is None) != (last_token is None) or (scatter is not None and scatter.numel() < R):
        raise KernelError("argmax: scatter and last_token go together, one scatter entry per row")
    _check(library().arle_argmax(_ptr(logits), logits.stride(0), R, V, _ptr(scratch), _ptr(out), _ptr(_i32(scatter, "scatter")),
                                 _ptr(_i32(last_token, "last_token")), _stream()), "argmax")
    add_launches(1)


def scatter_tokens(tokens, scatter, last_token) -> None:
    """last_token[scatter[r]] = tokens[r] (all int32), for tokens chosen by ``sample``."""
    R = scatter.numel()
    _i32(tokens, "tokens"), _i32(scatter, "scatter"), _i32(last_token, "last_token")
    if tokens.numel() < R:
        raise KernelError("scatter_tokens: one token per scatter entry")
    _check(library().arle_scatter_tokens(_ptr(tokens), _ptr(scatter), _ptr(last_token), R, _stream()), "scatter_tokens")


def sample(logits, temperature, top_k, top_p, min_p, uniform, scratch, out) -> None:
    """out[r] = next token of row r from float32 logits [R, V].  Per-row device
    arrays: temperature float32 (<= 0: greedy), top_k int32 (<= 0 off), top_p
    float32 (>= 1 off), min_p float32 (0 off), uniform float32 in [0, 1).  All of
    them None means every row is greedy.  scratch: float32 [R, V]."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with unit inner stride")
    if out.dtype != torch.int32 or out.numel() < R:
        raise KernelError("sample: out must be int32 with one entry per row")
    if temperature is not None:
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < R * V or not scratch.is_contiguous():
            raise KernelError("sample: scratch must be contiguous float32 [rows, vocab]")
        for t_, n_ in ((temperature, "temperature"), (top_p, "top_p"), (min_p, "min_p"), (uniform, "uniform")):
            if t_ is None or t_.dtype != torch.float32 or t_.numel() < R:
                raise KernelError(f"sample: {n_} must be float32 with one entry per row")
        _i32(top_k, "top_k")
    _check(library().arle_sample(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                 _ptr(min_p), _ptr(uniform), _ptr(scratch), _ptr(out), _stream()), "sample")
