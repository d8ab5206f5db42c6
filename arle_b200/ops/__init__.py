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
    "arle_embedding": [_P, _P, _I, _P, _I, _I, _I, _P, _P, _P, _F, _P],
    "arle_rmsnorm": [_P, _P, _P, _P, _P, _I, _I, _I, _F, _I, _P],
    "arle_residual_add": [_P, _P, _I, _I, _I, _P],
    "arle_silu_mul": [_P, _P, _I, _I, _I, _P],
    "arle_act_mul": [_P, _P, _I, _I, _I, _I, _I, _P],
    "arle_attention_prep_row": [_P, _I, _I, _P, _P, _P, _P, _F, _P, _P, _I, _I, _I, _P, _P, _I, _I, _I, _I, _I, _P],
    "arle_head_gate": [_P, _I, _P, _I, _F, _P, _I, _I, _I, _I, _I, _P],
    "arle_weighted_sum": [_P, _F, _P, _F, _P, _I, ctypes.c_longlong, _P],
    "arle_logit_cap": [_P, _F, ctypes.c_longlong, _P],
    "arle_gla_decay": [_P, _I, _I, _P, _P, _F, _P, _I, _I, _I, _P],
    "arle_gla_scan": [_P, _P, _P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P],
    "arle_gla_out": [_P, _P, _I, _I, _P, _F, _F, _P, _I, _I, _I, _I, _I, _P],
    "arle_attention_prep": [_P, _I, _I, _P, _P, _P, _P, _F, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P],
    "arle_rotary_angles": [_P, _P, _P, _I, _I, _P],
    "arle_paged_attention_plain": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _F, _I, _F, _I, _P],
    "arle_attention_prep_post": [_P, _I, _I, _P, _P, _P, _P, _F, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "arle_branch_norm_add": [_P, _P, _I, _P, _P, _I, _I, _I, _F, _P],
    "arle_branch_norm_add_norm": [_P, _P, _I, _P, _P, _P, _I, _I, _I, _F, _F, _P],
    "arle_rms_rows": [_P, _I, _I, _P, _P, _I, _I, _I, _I, _F, _P],
    "arle_normed_sum": [_P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _F, _P],
    "arle_bias_add": [_P, _I, _I, _P, _I, _I, _P],
    "arle_causal_conv": [_P, _I, _I, _P, _P, _P, _I, _P, ctypes.c_long, ctypes.c_long, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "arle_rglru_scan": [_P, _P, _P, _I, _I, _P, _P, _P, _P, _F, _P, ctypes.c_long, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "arle_delta_gates": [_P, _I, _P, _P, _P, _P, _I, _I, _P],
    "arle_delta_scan": [_P, _P, _P, _I, _I, _I, _I, _P, _P, _P, ctypes.c_long, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _P],
    "arle_clamped_glu": [_P, _P, _I, _I, _I, _I, _F, _F, _P],
    "arle_paged_attention_decode": [_P, _I, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _F, _I, _I, _I, _I, _F, _P],
    "arle_paged_attention_decode_stream": [_P, _I, _P, _P, _P, ctypes.c_longlong, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I,
                                           _F, _F, _I, _I, _I, _P, _P],
    "arle_paged_attention_decode_stream_prep": [_P, _I, _P, _P, _P, ctypes.c_longlong, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I,
                                                _F, _F, _I, _I, _I, _I, _P, _P, _P, _F, _P, _P, _P, _P],
    "arle_decode_stream_plan_ints": [_I, _I],
    "arle_decode_stream_plan": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "arle_paged_attention_prefill": [_P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _F, _I, _I, _I, _I, _I, _F, _P],
    "arle_paged_attention_prefill_tc": [_P, _I, _I, _P, _P, _P, ctypes.c_longlong, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _I,
                                        _I, _I, _I, _P, _I, _F, _P],
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
    "arle_dyt_norm": [_P, _P, _P, _P, _P, _F, _P, _I, _I, _I, _I, _P],
    "arle_gemm_heads_mma": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, ctypes.c_long, _I, _P],
    "arle_gemm_heads": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, ctypes.c_long, _I, _P],
    "arle_latent_prep": [_P, _I, _P, _I, _I, _P, _P, _P, _F, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P],
    "arle_latent_attention_mma": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P],
    "arle_latent_attention": [_P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "arle_decay_scan": [_P, _P, _P, _I, _I, _I, _I, _P, _P, _P, ctypes.c_long, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P],
    "arle_mlstm_gates": [_P, _I, _P, _P, _F, _P, _P, _P, ctypes.c_long, ctypes.c_long, _P, _P, _P, _I, _I, _P],
    "arle_mlstm_out": [_P, _P, _P, _I, _I, _P, _F, _P, _I, _I, _I, _I, _P],
    "arle_ssm_gates": [_P, _I, _P, _P, _P, _P, _I, _I, _P],
    "arle_conv_silu": [_P, _I, _I, _P, _P, _P, ctypes.c_long, ctypes.c_long, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "arle_gated_group_norm": [_P, _P, _I, _I, _P, _I, _P, _I, _P, _F, _P, _I, _I, _I, _I, _P],
    "arle_moe_select": [_P, _I, _P, _P, _I, _I, _I, _I, _F, _I, _P, _P, _I, _P],
    "arle_moe_plan": [_P, _I, _I, _I, _P, _P, _P, _P],
    "arle_moe_gemm": [_P, _I, _P, _P, _I, ctypes.c_long, _P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _P],
    "arle_moe_combine": [_P, _I, _P, _P, _I, _P, _I, _P, _I, _P, _I, _I, _I, _I, _P],
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
              last_token: torch.Tensor = None, slot_of_token: torch.Tensor = None, scale: float = 1.0) -> None:
    """out[t, :] = float32(table[ids[t], :]) * scale.  ids int32 [T]; out float32 [T, H].  With
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
                                    float(scale), _stream()), "embedding")


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


def gemm_tcgen05_pair(x, w, out, gated: bool = False, activation: str = "silu") -> None:
    """out[M, N] = x[M, K] . w[N, K]^T on the tcgen05 tensor cores with two SMs to a 256 x 256 tile
    (``cta_group::2``).  ``gated``: w holds (gate_i, up_i) in rows 2i and 2i + 1 and out [M, N / 2] gets
    act(gate) * up (``activation`` "silu" or "gelu_tanh"), the gate applied to the float32 sums in the kernel's
    epilogue."""
    M, K = x.shape
    N = w.shape[0]
    No = N // 2 if gated else N
    if (w.shape[1] != K or out.shape[0] != M or out.shape[1] != No or not tcgen05_gemm_supported(x, w, out)
            or (gated and (N % 2 or out.dtype != torch.bfloat16))):
        raise KernelError(f"gemm_tcgen05_pair: unsupported operands x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    _check(library().arle_gemm_tcgen05_pair(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), _dt(out), out.stride(0), M,
                                            N, K, (1 + ACTIVATIONS[activation]) if gated else 0, _ptr(error_flag(x.device)),
                                            _stream()), "gemm_tcgen05_pair")


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
                    page_size: int, scale: float, window, batch=None, vd: int = None, sink: float = None, keep_first: int = 0,
                    softcap: float = None) -> None:
    """Causal attention of this step's queries over the paged cache.

    ``keep_first``: with a window, the keys j < keep_first stay visible (at their true places) after the window has
    passed them.  ``softcap``: a score s becomes softcap * tanh(s / softcap) before the softmax.

    ``vd``: the values' width when it differs from the keys' (the value cache is then [pages, nkv, page_size, vd] and
    out [T, nq*vd]).  ``sink``: the score of a sink without a value that the softmax's denominator counts besides the
    keys, p_j = exp(s_j) / (exp(sink) + sum exp(s_j)); None for the usual softmax.  Values of another width run on the
    general kernel; the sink is one more term at the end of every kernel's sums.

    q: [T, nq*hd] view (row stride free, unit inner stride); out: contiguous
    [T, nq*hd]; caches [pages, nkv, page_size, hd]; positions / row_of_token int32
    [T]; block_table int32 [rows, max_pages].  ``window`` None or <= 0 means all
    keys.  ``batch`` (a StepContext) lets faster kernels pick their launch shape;
    the general kernel does not need it."""
    T = q.shape[0]
    vd = hd if vd is None else int(vd)
    if q.stride(1) != 1 or q.shape[1] != nq * hd or out.shape != (T, nq * vd) or not out.is_contiguous():
        raise KernelError("paged_attention: q must be [T, nq*hd] with unit inner stride and out contiguous [T, nq*vd]")
    if q.dtype != k_cache.dtype or out.dtype != q.dtype:
        raise KernelError("paged_attention: q, out and cache must share a type")
    if hd > 256 or vd > 256 or nq % nkv:
        raise KernelError(f"paged_attention: head_dim {hd} / value width {vd} / heads {nq}:{nkv} not supported")
    if (tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or tuple(v_cache.shape[1:]) != (nkv, page_size, vd)
            or not k_cache.is_contiguous() or not v_cache.is_contiguous()):
        raise KernelError(f"paged_attention: cache shapes {tuple(k_cache.shape)}, {tuple(v_cache.shape)} are not "
                          f"[pages, {nkv}, {page_size}, {hd}] and [pages, {nkv}, {page_size}, {vd}]")
    _i32(positions, "positions"), _i32(row_of_token, "row_of_token"), _i32(block_table, "block_table")
    if block_table.stride(1) != 1:
        raise KernelError("paged_attention: block table rows must be contiguous")
    keep_first = int(keep_first or 0) if window else 0
    if batch is not None and _KERNEL_SET == "fast" and vd == hd and fast_attention_supported(q, nq, nkv, hd):
        # kept first keys and capped scores are in both prompt kernels and in the split-KV decode kernel (not the streaming one)
        extended = bool(keep_first or softcap)
        if batch.max_q_len > 1:
            prefill = paged_attention_prefill_tc if tc_attention_supported(q, hd, page_size) else paged_attention_prefill
            prefill(q, out, k_cache, v_cache, batch.q_indptr, batch.kv_lens, block_table, nq, nkv, hd, page_size, scale,
                    window, batch.max_q_len, skip_single=batch.num_single > 0, sink=sink, keep_first=keep_first, softcap=softcap)
        if batch.num_single > 0 and not extended and stream_decode_supported(batch.num_rows, page_size, nq // nkv):
            ctas = sm_count(q.device)
            slots = (ctas + batch.num_rows * nkv) * (nq // nkv)
            paged_attention_decode_stream(
                q, out, k_cache, v_cache, batch.q_indptr, batch.kv_lens, block_table, nq, nkv, hd, page_size, scale, window,
                batch.ws.get("attn_piece_o", (slots * hd,), torch.float32),
                batch.ws.get("attn_piece_ml", (slots * 2,), torch.float32),
                batch.ws.get_zeroed("attn_piece_counters", (batch.num_rows * nkv,), torch.int32), ctas, sink=sink)
        elif batch.num_single > 0:
            bound = block_table.shape[1] * page_size
            if window:
                bound = min(bound, int(window) + keep_first + 63)
            splits = decode_splits(batch.num_rows, nkv, bound, q.device)
            part_o = part_ml = counters = None
            if splits > 1:
                part_o = batch.ws.get("attn_part_o", (batch.num_rows * nq * splits * hd,), torch.float32)
                part_ml = batch.ws.get("attn_part_ml", (batch.num_rows * nq * splits * 2,), torch.float32)
                counters = batch.ws.get_zeroed("attn_split_counters", (batch.num_rows * nkv,), torch.int32)
            paged_attention_decode(q, out, k_cache, v_cache, batch.q_indptr, batch.kv_lens, block_table, nq, nkv, hd,
                                   page_size, scale, window, splits, part_o, part_ml, counters, sink=sink, keep_first=keep_first,
                                   softcap=softcap)
        return
    _check(library().arle_paged_attention_plain(
        _ptr(q), q.stride(0), _ptr(out), _ptr(k_cache), _ptr(v_cache), _dt(q), _ptr(positions), _ptr(row_of_token),
        _ptr(block_table), block_table.stride(0), nq, nkv, hd, vd, page_size, float(scale),
        int(window) if window else 0, int(sink is not None), float(sink or 0.0), keep_first, float(softcap or 0.0), T, _stream()),
        "paged_attention")


def _sink_arg(sink) -> float:
    """The fast attention kernels take the sink's score as a number; minus infinity stands for no sink (its term is zero)."""
    return float("-inf") if sink is None else float(sink)


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
                               window, max_q_len: int, skip_single: bool = False, sink: float = None, keep_first: int = 0,
                               softcap: float = None) -> None:
    """Flash attention over the paged cache on the tcgen05 tensor cores (TMA-fed, scores
    and output in tensor memory) for rows with several queries."""
    R = kv_lens.numel()
    _i32(q_indptr, "q_indptr"), _i32(kv_lens, "kv_lens"), _i32(block_table, "block_table")
    if not tc_attention_supported(q, hd, page_size) or q.stride(1) != 1 or not out.is_contiguous():
        raise KernelError("paged_attention_prefill_tc: needs bfloat16, head size 128, page size a multiple of 16")
    _check(library().arle_paged_attention_prefill_tc(
        _ptr(q), q.stride(0), q.shape[0], _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(q_indptr),
        _ptr(kv_lens), _ptr(block_table), block_table.stride(0), block_table.shape[1], nq, nkv, hd, page_size, float(scale),
        _sink_arg(sink), int(window) if window else 0, R, int(max_q_len), int(bool(skip_single)), _ptr(error_flag(q.device)),
        int(keep_first or 0), float(softcap or 0.0), _stream()), "paged_attention_prefill_tc")


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
                                  window, piece_o, piece_ml, counters, ctas: int, sink: float = None) -> None:
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
        nq, nkv, hd, page_size, float(scale), _sink_arg(sink), int(window) if window else 0, R, int(ctas), _ptr(error_flag(q.device)),
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
        _ptr(counters), nq, nkv, hd, page_size, float(scale), _sink_arg(None), int(window) if window else 0, R, int(ctas), 1,
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
                           window, splits: int, part_o=None, part_ml=None, counters=None, sink: float = None, keep_first: int = 0,
                           softcap: float = None) -> None:
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
        float(scale), _sink_arg(sink), int(window) if window else 0, R, int(splits), int(keep_first or 0), float(softcap or 0.0),
        _stream()), "paged_attention_decode")


def paged_attention_prefill(q, out, k_cache, v_cache, q_indptr, kv_lens, block_table, nq, nkv, hd, page_size, scale,
                            window, max_q_len: int, skip_single: bool = False, sink: float = None, keep_first: int = 0,
                            softcap: float = None) -> None:
    """Flash-attention over the paged cache for rows with several queries (and,
    unless skip_single, for single-query rows too)."""
    R = kv_lens.numel()
    _i32(q_indptr, "q_indptr"), _i32(kv_lens, "kv_lens"), _i32(block_table, "block_table")
    _check(library().arle_paged_attention_prefill(
        _ptr(q), q.stride(0), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(q_indptr), _ptr(kv_lens),
        _ptr(block_table), block_table.stride(0), nq, nkv, hd, page_size, float(scale),
        _sink_arg(sink), int(window) if window else 0, R, int(max_q_len), int(bool(skip_single)), int(keep_first or 0),
        float(softcap or 0.0), _stream()), "paged_attention_prefill")


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


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out[t, i] = act(gate_up[t, 2i]) * gate_up[t, 2i + 1] for ``activation`` "silu" or "gelu_tanh" (the tanh
    form of gelu); float32 arithmetic, rounded once.  ``out`` may be columns of a wider buffer."""
    T, I = out.shape
    if activation not in ACTIVATIONS:
        raise KernelError(f"act_mul: activation {activation!r} (known: {', '.join(ACTIVATIONS)})")
    if gate_up.shape != (T, 2 * I) or not gate_up.is_contiguous() or out.stride(1) != 1 or gate_up.dtype != out.dtype:
        raise KernelError("act_mul: gate_up must be contiguous [T, 2I] and out [T, I] of the same type with unit inner stride")
    _check(library().arle_act_mul(_ptr(gate_up), _ptr(out), _dt(out), T, I, ACTIVATIONS[activation], out.stride(0) if T > 1 else I,
                                  _stream()), "act_mul")


def gemm_act_mul(x, w: torch.Tensor, gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """The first half of a gated feed-forward with the named activation on the gate (any of ``ACTIVATIONS``):
    out[t, i] = act(x[t] . w[2i]) * (x[t] . w[2i + 1]).  ``out`` may be columns of a wider buffer.  Few rows of x
    take one launch of the weight-streaming kernel (``x`` may then be ``ScaledRows``), many rows one launch of the
    two-SM tcgen05 kernel, the gate applied to the float32 sums; otherwise the product goes to ``gate_up`` [T, 2I]
    and the gate kernel follows."""
    if activation not in ACTIVATIONS:
        raise KernelError(f"gemm_act_mul: activation {activation!r} (known: {', '.join(ACTIVATIONS)})")
    if activation == "silu" and out.is_contiguous():
        gemm_silu_mul(x, w, gate_up, out)
        return
    T, I = out.shape
    if w.shape[0] != 2 * I or gate_up.shape != (T, 2 * I) or out.stride(1) != 1:
        raise KernelError(f"gemm_act_mul: shapes w {tuple(w.shape)} gate_up {tuple(gate_up.shape)} out {tuple(out.shape)}")
    code = 1 + ACTIVATIONS[activation]
    if isinstance(x, ScaledRows):
        if not (fused_gemm_supported(x.rows, w) and gated_gemm_fits(x.rows.shape[1])):
            raise KernelError("gemm_act_mul: rows that lack their norm factor need the gated weight-streaming kernel")
        _fused_gemm(x.rows, w, out, code, x, None)
        return
    if (_KERNEL_SET == "fast" and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and fused_gemm_supported(x, w) and skinny_gemm_supported(x, w, out) and gated_gemm_fits(x.shape[1])):
        _fused_gemm(x, w, out, code, None, None)
        return
    if (_KERNEL_SET == "fast" and T >= _GATED_TCGEN05_MIN_ROWS and x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and tcgen05_gemm_supported(x, w, out) and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0):
        gemm_tcgen05_pair(x, w, out, gated=True, activation=activation)
        return
    gemm(x, w, gate_up)
    act_mul(gate_up, out, activation)


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


# ------------------------------------------------- attention with a norm over the whole row
ROTARY_PAIRINGS = {"half": 0, "interleaved": 1}


def attention_prep_row(qk, positions, slot_mapping, q_weight, k_weight, eps: float, inv_freq, rotary_dim: int, pairing: str,
                       values_are_keys: bool, k_cache, v_cache, nq: int, nkv: int, hd: int, page_size: int, angles=None) -> None:
    """RMSNorm of q and of k over their whole projected rows (weights float32 [nq*hd], [nkv*hd], or None: no
    norm), rotation of the first ``rotary_dim`` elements of every head (``pairing`` "half": element i with
    i + rotary_dim/2; "interleaved": 2i with 2i + 1), q stored in place on qk [T, >= (nq + nkv) hd], k into the
    paged k_cache; v_cache gets the keys as projected (``values_are_keys``) or the v heads that follow the k
    heads in the row.  nkv = 0: queries only, nothing stored.  ``angles``: the table of ``rotary_angles`` for these
    positions and inv_freq (float32 [T, rotary_dim / 2, 2]), or None: the kernel evaluates them itself (the same bits)."""
    T = qk.shape[0]
    if angles is not None and (angles.dtype != torch.float32 or tuple(angles.shape) != (T, rotary_dim // 2, 2)
                               or not angles.is_contiguous()):
        raise KernelError("attention_prep_row: angles must be contiguous float32 [T, rotary_dim / 2, 2]")
    need = (nq + (nkv if values_are_keys else 2 * nkv)) * hd
    if qk.stride(1) != 1 or qk.shape[1] < need:
        raise KernelError(f"attention_prep_row: qk must be [T, >= {need}] with unit inner stride")
    if pairing not in ROTARY_PAIRINGS:
        raise KernelError(f"attention_prep_row: pairing {pairing!r} (known: {', '.join(ROTARY_PAIRINGS)})")
    for w_, n_ in ((q_weight, nq * hd), (k_weight, nkv * hd)):
        if w_ is not None and (w_.dtype != torch.float32 or w_.numel() != n_ or not w_.is_contiguous()):
            raise KernelError("attention_prep_row: norm weights must be contiguous float32 over the whole row")
    if nkv > 0:
        if k_cache.dtype != qk.dtype or v_cache.dtype != qk.dtype:
            raise KernelError("attention_prep_row: cache type differs from activation type")
        if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or k_cache.shape != v_cache.shape or not (
                k_cache.is_contiguous() and v_cache.is_contiguous()):
            raise KernelError(f"attention_prep_row: cache shape {tuple(k_cache.shape)} is not [pages, {nkv}, {page_size}, {hd}]")
        _i32(slot_mapping, "slot_mapping")
    _i32(positions, "positions")
    if rotary_dim and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("attention_prep_row: inv_freq must be float32 [rotary_dim / 2]")
    _check(library().arle_attention_prep_row(
        _ptr(qk), _dt(qk), qk.stride(0), _ptr(positions), _ptr(slot_mapping) if nkv else None, _ptr(q_weight), _ptr(k_weight),
        float(eps), _ptr(inv_freq) if rotary_dim else None, _ptr(angles) if rotary_dim else None, int(rotary_dim),
        ROTARY_PAIRINGS[pairing], int(bool(values_are_keys)),
        _ptr(k_cache) if nkv else None, _ptr(v_cache) if nkv else None, nq, nkv, hd, page_size, T, _stream()),
        "attention_prep_row")


def head_gate(x, gate, scale: float, out, heads: int, hd: int) -> None:
    """out[t, h*hd + e] = x[t, h*hd + e] * sigmoid(gate[t, h]) * scale (gate None: no gate, a scaled copy).
    x [T, heads*hd], gate [T, heads] and out [T, heads*hd] may be slices of wider rows (unit inner stride)."""
    T = x.shape[0]
    if (x.shape[1] != heads * hd or out.shape != (T, heads * hd) or x.dtype != out.dtype or x.stride(1) != 1
            or out.stride(1) != 1 or (gate is not None and (gate.shape != (T, heads) or gate.dtype != out.dtype
                                                            or gate.stride(1) != 1))):
        raise KernelError(f"head_gate: shapes x {tuple(x.shape)} out {tuple(out.shape)} or the gate's do not fit")
    _check(library().arle_head_gate(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, float(scale),
                                    _ptr(out), out.stride(0), _dt(out), T, heads, hd, _stream()), "head_gate")


def weighted_sum(x, a: float, y, b: float, out) -> None:
    """out = a * x + b * y (float32 arithmetic, rounded once); contiguous tensors of one shape and type."""
    if x.shape != y.shape or x.shape != out.shape or x.dtype != y.dtype or x.dtype != out.dtype or not (
            x.is_contiguous() and y.is_contiguous() and out.is_contiguous()):
        raise KernelError("weighted_sum: x, y and out must be contiguous and of one shape and type")
    _check(library().arle_weighted_sum(_ptr(x), float(a), _ptr(y), float(b), _ptr(out), _dt(out), x.numel(), _stream()),
           "weighted_sum")


def logit_cap(logits, cap: float) -> None:
    """logits <- cap * tanh(logits / cap), in place; contiguous float32."""
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("logit_cap: logits must be contiguous float32")
    _check(library().arle_logit_cap(_ptr(logits), float(cap), logits.numel(), _stream()), "logit_cap")


# ------------------------------------------------------------ gated linear attention
def gla_decay(low, w2t, bias, tau: float, alpha) -> None:
    """alpha[t, c] = sigmoid(bias[c] + sum_r low[t, r] * w2t[r, c]) ^ (1 / tau), float32 [T, channels].  ``low``
    [T, rank] in the activation type (a slice of a wider row is fine), w2t float32 [rank, channels] (the gate's
    second matrix transposed), bias float32 [channels] or None."""
    T, rank = low.shape
    C = w2t.shape[1]
    w2 = w2t
    if (w2.dtype != torch.float32 or w2.shape[0] != rank or not w2.is_contiguous() or alpha.dtype != torch.float32
            or tuple(alpha.shape) != (T, C) or not alpha.is_contiguous() or low.stride(1) != 1):
        raise KernelError(f"gla_decay: shapes low {tuple(low.shape)} w2t {tuple(w2.shape)} alpha {tuple(alpha.shape)}")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != C):
        raise KernelError("gla_decay: bias must be float32 [channels]")
    _check(library().arle_gla_decay(_ptr(low), _dt(low), low.stride(0), _ptr(w2), _ptr(bias), float(tau), _ptr(alpha), T, C,
                                    rank, _stream()), "gla_decay")


def gla_scan(q, k, v, alpha, state, q_indptr, state_slots, out, heads: int, dim: int, vdim: int, q_scale: float,
             max_q_len: int) -> None:
    """The recurrence S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T (q_t * q_scale) over the tokens of every row of
    the step (row r owns tokens q_indptr[r] .. q_indptr[r+1]-1), from and into state[state_slots[r]].
    q, k [T, heads*dim] and v [T, heads*vdim]: slices of one wider buffer (same row stride, unit inner stride);
    alpha float32 [T, heads*dim]; state float32 [slots, heads, vdim, dim] (a head's state transposed);
    out float32 [T, heads*vdim]."""
    T = q.shape[0]
    R = state_slots.numel()
    if (q.shape != (T, heads * dim) or k.shape != q.shape or v.shape != (T, heads * vdim) or q.dtype != k.dtype
            or q.dtype != v.dtype or q.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1
            or q.stride(0) != k.stride(0) or q.stride(0) != v.stride(0)):
        raise KernelError("gla_scan: q, k, v must be slices of one buffer: [T, heads*dim], [T, heads*dim], [T, heads*vdim]")
    if alpha.dtype != torch.float32 or tuple(alpha.shape) != (T, heads * dim) or not alpha.is_contiguous():
        raise KernelError("gla_scan: alpha must be contiguous float32 [T, heads*dim]")
    if (state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, vdim, dim) or not state.is_contiguous()):
        raise KernelError(f"gla_scan: state {tuple(state.shape)} is not float32 [slots, {heads}, {vdim}, {dim}]")
    if out.dtype != torch.float32 or tuple(out.shape) != (T, heads * vdim) or not out.is_contiguous():
        raise KernelError("gla_scan: out must be contiguous float32 [T, heads*vdim]")
    _i32(q_indptr, "q_indptr"), _i32(state_slots, "state_slots")
    if q_indptr.numel() != R + 1:
        raise KernelError("gla_scan: q_indptr must have one entry more than state_slots")
    _check(library().arle_gla_scan(_ptr(q), _ptr(k), _ptr(v), _dt(q), q.stride(0), _ptr(alpha), _ptr(state), _ptr(q_indptr),
                                   _ptr(state_slots), _ptr(out), R, heads, dim, vdim, float(q_scale), int(max_q_len), _stream()),
           "gla_scan")


def gla_out(o, gate, weight, eps: float, scale: float, out, heads: int, vdim: int, gate_act: str = "silu") -> None:
    """out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * silu(gate[t, h, :]) * scale (``gate_act`` "sigmoid": times
    sigmoid(gate) instead).
    o float32 [T, heads*vdim] contiguous; gate (activation type, or None) and out may be slices of wider rows;
    weight float32 [vdim] or None."""
    T = o.shape[0]
    if o.dtype != torch.float32 or tuple(o.shape) != (T, heads * vdim) or not o.is_contiguous():
        raise KernelError("gla_out: o must be contiguous float32 [T, heads*vdim]")
    if out.shape != o.shape or out.stride(1) != 1 or (gate is not None and (gate.shape != o.shape or gate.stride(1) != 1
                                                                          or gate.dtype != out.dtype)):
        raise KernelError("gla_out: gate and out must be [T, heads*vdim] of one type with unit inner stride")
    if weight is not None and (weight.dtype != torch.float32 or weight.numel() != vdim):
        raise KernelError("gla_out: weight must be float32 [vdim]")
    if gate_act not in ("silu", "sigmoid"):
        raise KernelError(f"gla_out: gate_act {gate_act!r} (silu, sigmoid)")
    _check(library().arle_gla_out(_ptr(o), _ptr(gate), _dt(out), gate.stride(0) if gate is not None else 0, _ptr(weight),
                                  float(eps), float(scale), _ptr(out), out.stride(0), T, heads, vdim, int(gate_act == "sigmoid"), _stream()),
           "gla_out")


# ------------------------------------------------------------------ a norm without statistics
def dyt_norm(resid, delta, rows, weight, bias, alpha: float, out, write_resid: bool) -> None:
    """Dynamic Tanh in a norm's place, with the residual sum of ``rmsnorm`` in front of it: for output row i (source
    row r = rows[i], or i) x = resid[r] (+ delta[r]); resid[r] = x when write_resid; out[i] = tanh(alpha * x) * weight
    + bias.  resid float32 [N, H]; delta and out in the activation type; weight, bias float32 [H] (bias may be None)."""
    H = resid.shape[1]
    n_out = out.shape[0]
    if resid.dtype != torch.float32 or weight.dtype != torch.float32 or (bias is not None and bias.dtype != torch.float32):
        raise KernelError("dyt_norm: residual, weight and bias must be float32")
    if not (resid.is_contiguous() and out.is_contiguous()) or out.shape[1] != H or weight.numel() != H or (
            bias is not None and bias.numel() != H):
        raise KernelError("dyt_norm: bad shapes or strides")
    if delta is not None and (delta.dtype != out.dtype or delta.shape != resid.shape or not delta.is_contiguous()):
        raise KernelError("dyt_norm: delta must match the residual's shape and the output's type")
    if rows is not None:
        _i32(rows, "rows")
        if rows.numel() != n_out:
            raise KernelError("dyt_norm: one output row per entry of rows")
    elif n_out != resid.shape[0]:
        raise KernelError("dyt_norm: output rows must match residual rows when no row list is given")
    _check(library().arle_dyt_norm(_ptr(resid), _ptr(delta), _ptr(rows), _ptr(weight), _ptr(bias), float(alpha), _ptr(out), _dt(out),
                                   n_out, H, int(bool(write_resid)), _stream()), "dyt_norm")


# ------------------------------------------------------------------ attention over latent vectors
def gemm_heads(x, w, out) -> None:
    """out[m, h, :] = x[m, h, :] . w[h]^T for every head h: x [M, heads, K], w [heads, N, K] contiguous, out [M, heads, N].
    x and out may be views into wider rows (any row stride and head stride, unit inner stride).  float32 sums; k ascending
    in the general kernel, tensor-core tiles for bfloat16 rows on 16-byte boundaries (fast kernel set).  ``out`` has x's
    type, or is float32 (the sums as they are) for bfloat16 rows."""
    M, heads, K = x.shape
    N = w.shape[1]
    if (w.shape[0] != heads or w.shape[2] != K or tuple(out.shape) != (M, heads, N) or not w.is_contiguous()
            or x.stride(2) != 1 or out.stride(2) != 1 or (x.dtype != out.dtype and out.dtype != torch.float32)):
        raise KernelError(f"gemm_heads: shapes x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    if x.dtype == torch.bfloat16 and w.dtype != torch.bfloat16:
        raise KernelError("gemm_heads: bfloat16 rows need bfloat16 matrices")
    if (_KERNEL_SET == "fast" and x.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        # the same sums on the tensor cores (tiles of 64 rows x 128 columns)
        _check(library().arle_gemm_heads_mma(_ptr(x), _ptr(w), _ptr(out), _dt(out), M, N, K, heads, x.stride(0), K, out.stride(0), x.stride(1),
                                             N * K, out.stride(1), _stream()), "gemm_heads_mma")
        return
    _check(library().arle_gemm_heads(_ptr(x), _ptr(w), _ptr(out), _dt(x), _dt(w), _dt(out), M, N, K, heads, x.stride(0), K, out.stride(0),
                                     x.stride(1), N * K, out.stride(1), _stream()), "gemm_heads")


def latent_prep(q, dkv, positions, slot_mapping, c_weight, eps: float, inv_freq, rot_dims: int, cache, q_abs, heads: int,
                dn: int, dr: int, rank: int) -> None:
    """The per-token preparation of an attention whose cache holds one record [latent | rotated key part] per token.
    dkv [T, >= rank + dr]: its first ``rank`` numbers are RMS-normed with ``c_weight`` (float32 [rank]), its next ``dr``
    numbers are rotated (the first ``rot_dims`` of them, element i with i + rot_dims / 2, by position * inv_freq[i]);
    both go to cache[slot_mapping[t]] (cache [pages, 1, page_size, rank + dr]; None: nothing is stored).  q [T, >= heads
    * (dn + dr)]: every head's last ``dr`` numbers are rotated the same way into q_abs[t, h, rank:] (q_abs [T, heads,
    rank + dr], contiguous)."""
    T = q.shape[0]
    kd = rank + dr
    if cache is None and dkv is None:               # nothing to store: only the queries' rotated numbers are prepared
        dkv, c_weight = q, None
    elif dkv is None or c_weight is None:
        raise KernelError("latent_prep: a cache to store into needs dkv and the latent's norm weight")
    if (q.stride(1) != 1 or dkv.stride(1) != 1 or q.shape[1] < heads * (dn + dr) or (cache is not None and dkv.shape[1] < kd)
            or q.dtype != dkv.dtype or tuple(q_abs.shape) != (T, heads, kd) or not q_abs.is_contiguous() or q_abs.dtype != q.dtype):
        raise KernelError("latent_prep: q, dkv or q_abs do not fit the sizes given")
    if c_weight is not None and (c_weight.dtype != torch.float32 or c_weight.numel() != rank):
        raise KernelError("latent_prep: the latent's norm weight must be float32 [rank]")
    if rot_dims and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2):
        raise KernelError("latent_prep: inv_freq must be float32 [rot_dims / 2]")
    if cache is not None:
        if cache.dtype != q.dtype or cache.shape[1] != 1 or cache.shape[3] != kd or not cache.is_contiguous():
            raise KernelError(f"latent_prep: cache shape {tuple(cache.shape)} is not [pages, 1, page_size, {kd}] of the activation type")
        _i32(slot_mapping, "slot_mapping")
    _i32(positions, "positions")
    _check(library().arle_latent_prep(_ptr(q), q.stride(0), _ptr(dkv), dkv.stride(0), _dt(q), _ptr(positions),
                                      _ptr(slot_mapping) if cache is not None else None, _ptr(c_weight), float(eps),
                                      _ptr(inv_freq) if rot_dims else None, int(rot_dims), _ptr(cache), _ptr(q_abs), heads, dn, dr,
                                      rank, T, _stream()), "latent_prep")


def latent_mma_supported(q_abs, rank: int) -> bool:
    """The tensor-core latent attention takes bfloat16, a latent of 64, 128, 256 or 512 and a rotated part that is a multiple
    of 16; everything else runs on the general kernel."""
    kd = q_abs.shape[2]
    return (_KERNEL_SET == "fast" and q_abs.dtype == torch.bfloat16 and rank in (64, 128, 256, 512) and (kd - rank) % 16 == 0
            and q_abs.data_ptr() % 16 == 0)


def latent_attention(q_abs, out, cache, positions, row_of_token, block_table, rank: int, page_size: int, scale: float, window,
                     batch=None) -> None:
    """Causal attention of folded queries q_abs [T, heads, kd] over records cache [pages, 1, page_size, kd]: head h's score
    against record j is (q_abs[t, h] . record_j) * scale, its output sum_j softmax_j * record_j[:rank] (out [T, heads,
    rank]).  ``window`` None or <= 0: all keys; W: keys p - W + 1 .. p.  Scores, softmax and sums are float32.  ``batch`` (a
    StepContext, for its scratch buffers) lets the tensor-core kernel run where the shapes allow it; with few tokens in
    the step a token's keys are shared out among several blocks."""
    T, heads, kd = q_abs.shape
    if (not q_abs.is_contiguous() or tuple(out.shape) != (T, heads, rank) or not out.is_contiguous() or out.dtype != q_abs.dtype
            or cache.dtype != q_abs.dtype or tuple(cache.shape[1:]) != (1, page_size, kd) or not cache.is_contiguous()):
        raise KernelError("latent_attention: q_abs [T, heads, kd], out [T, heads, rank] and cache [pages, 1, page_size, kd] of one type")
    _i32(positions, "positions"), _i32(row_of_token, "row_of_token"), _i32(block_table, "block_table")
    if block_table.stride(1) != 1:
        raise KernelError("latent_attention: block table rows must be contiguous")
    if batch is not None and latent_mma_supported(q_abs, rank):
        bound = block_table.shape[1] * page_size
        if window:
            bound = min(bound, int(window) + 63)
        blocks = T * (-(-heads // 16))
        splits = max(1, min(-(-bound // 64), -(-4 * sm_count(q_abs.device) // blocks), 64))
        part_o = part_ml = None
        if splits > 1:
            part_o = batch.ws.get("latent_part_o", (T * heads * splits * rank,), torch.float32)
            part_ml = batch.ws.get("latent_part_ml", (T * heads * splits * 2,), torch.float32)
        _check(library().arle_latent_attention_mma(_ptr(q_abs), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(cache), _ptr(positions),
                                                   _ptr(row_of_token), _ptr(block_table), block_table.stride(0), heads, rank, kd,
                                                   page_size, float(scale), int(window) if window else 0, T, splits, _stream()),
               "latent_attention_mma")
        if splits > 1:
            add_launches(1)
        return
    _check(library().arle_latent_attention(_ptr(q_abs), _ptr(out), _ptr(cache), _dt(q_abs), _ptr(positions), _ptr(row_of_token),
                                           _ptr(block_table), block_table.stride(0), heads, rank, kd, page_size, float(scale),
                                           int(window) if window else 0, T, _stream()), "latent_attention")


# ------------------------------------------------------------------ matrix memories with a scalar decay
def decay_scan(q, k, v, a, b, state, q_indptr, state_slots, out, heads: int, kq_heads: int, dim: int, vdim: int,
               ones_column: bool, q_scale: float, act: str = "none") -> None:
    """S_t = a_t S_(t-1) + b_t k_t v_t^T, o_t = S_t^T (q_t * q_scale) over the tokens of every row of the step (row r owns
    tokens q_indptr[r] .. q_indptr[r+1]-1), from and into state[state_slots[r]].  q, k [T, kq_heads*dim] (head h reads
    head h // (heads / kq_heads)), v [T, heads*vdim], in the activation type (views of wider rows are fine); a, b float32
    [T, heads]; state float32 [slots, n] whose first heads * vcols * dim numbers are the memories, a head's transposed
    ([heads][vcols][dim]); vcols = vdim + 1 with ``ones_column`` (a column of ones beside v: it carries sum a..b k, the
    normaliser of a matrix LSTM); out float32 [T, heads, vcols].  A memory whose decay is one constant per head gives a as
    float32 [heads] and b as float32 [heads] or None (ones).  ``act`` "silu": q, k and v go through silu as the kernel
    reads them."""
    T = v.shape[0]
    R = state_slots.numel()
    vcols = vdim + int(bool(ones_column))
    if (q.shape != (T, kq_heads * dim) or k.shape != q.shape or v.shape != (T, heads * vdim) or q.dtype != k.dtype
            or q.dtype != v.dtype or q.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1):
        raise KernelError("decay_scan: q, k [T, kq_heads*dim] and v [T, heads*vdim] of one type with unit inner stride")
    per_head = a.dim() == 1
    if act not in ("none", "silu"):
        raise KernelError(f"decay_scan: act {act!r} (none, silu)")
    for t_, n_ in ((a, "a"), (b, "b")):
        if t_ is None and per_head and n_ == "b":
            continue
        if t_ is None or t_.dtype != torch.float32 or tuple(t_.shape) != ((heads,) if per_head else (T, heads)) or not t_.is_contiguous():
            raise KernelError(f"decay_scan: {n_} must be contiguous float32 [T, heads] (or [heads] for both)")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < heads * vcols * dim or state.stride(1) != 1:
        raise KernelError(f"decay_scan: state {tuple(state.shape)} must be float32 [slots, >= {heads * vcols * dim}]")
    if out.dtype != torch.float32 or tuple(out.shape) != (T, heads, vcols) or not out.is_contiguous():
        raise KernelError("decay_scan: out must be contiguous float32 [T, heads, vcols]")
    _i32(q_indptr, "q_indptr"), _i32(state_slots, "state_slots")
    if q_indptr.numel() != R + 1:
        raise KernelError("decay_scan: q_indptr must have one entry more than state_slots")
    _check(library().arle_decay_scan(_ptr(q), _ptr(k), _ptr(v), _dt(q), q.stride(0), k.stride(0), v.stride(0), _ptr(a), _ptr(b),
                                     _ptr(state), state.stride(0), _ptr(q_indptr), _ptr(state_slots), _ptr(out), R, heads, kq_heads,
                                     dim, vdim, vcols - vdim, float(q_scale), 0 if per_head else heads, int(act == "silu"), int(T > 16 * R),
                                     _stream()),
           "decay_scan")


def mlstm_gates(pre, bias_i, bias_f, cap: float, q_indptr, state_slots, state, m_offset: int, a, b, floor) -> None:
    """The gates of a matrix LSTM.  pre float32 [T, 2*heads]: the input gates' sums, then the forget gates'.  Per head
    i = cap tanh((pre_i + bias_i) / cap), f = logsigmoid(cap tanh((pre_f + bias_f) / cap)), the running maximum
    m_t = max(f + m_(t-1), i) (m of request slot s at state[s, m_offset + head]; it starts at what the slot holds, zero
    for a new request, and is left at the row's last value), and a = exp(f + m_(t-1) - m_t), b = exp(i - m_t),
    floor = exp(-m_t), all float32 [T, heads]."""
    T = pre.shape[0]
    heads = pre.shape[1] // 2
    R = state_slots.numel()
    if pre.dtype != torch.float32 or pre.stride(1) != 1 or pre.shape[1] != 2 * heads:
        raise KernelError("mlstm_gates: pre must be float32 [T, 2*heads] with unit inner stride")
    for t_ in (a, b, floor):
        if t_.dtype != torch.float32 or tuple(t_.shape) != (T, heads) or not t_.is_contiguous():
            raise KernelError("mlstm_gates: a, b and floor must be contiguous float32 [T, heads]")
    for t_ in (bias_i, bias_f):
        if t_ is not None and (t_.dtype != torch.float32 or t_.numel() != heads):
            raise KernelError("mlstm_gates: biases must be float32 [heads]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < m_offset + heads or state.stride(1) != 1:
        raise KernelError("mlstm_gates: state must be float32 [slots, n] and hold the maxima at m_offset")
    _i32(q_indptr, "q_indptr"), _i32(state_slots, "state_slots")
    _check(library().arle_mlstm_gates(_ptr(pre), pre.stride(0), _ptr(bias_i), _ptr(bias_f), float(cap), _ptr(q_indptr),
                                      _ptr(state_slots), _ptr(state), state.stride(0), int(m_offset), _ptr(a), _ptr(b), _ptr(floor),
                                      R, heads, _stream()), "mlstm_gates")


def mlstm_out(num, floor, gate, weight, eps: float, out, heads: int, vdim: int) -> None:
    """out[t, h, :] = rms_unit(num[t, h, :vdim] / (max(|num[t, h, vdim]|, floor[t, h]) + 1e-6)) * weight[h, :] *
    sigmoid(gate[t, h, :]).  num float32 [T, heads, vdim + 1] (what ``decay_scan`` leaves with its column of ones);
    gate and out [T, heads*vdim] in the activation type (views of wider rows are fine); weight float32 [heads*vdim]."""
    T = num.shape[0]
    if num.dtype != torch.float32 or tuple(num.shape) != (T, heads, vdim + 1) or not num.is_contiguous():
        raise KernelError("mlstm_out: num must be contiguous float32 [T, heads, vdim + 1]")
    if (floor.dtype != torch.float32 or tuple(floor.shape) != (T, heads) or not floor.is_contiguous()
            or weight.dtype != torch.float32 or weight.numel() != heads * vdim):
        raise KernelError("mlstm_out: floor float32 [T, heads], weight float32 [heads*vdim]")
    if (tuple(out.shape) != (T, heads * vdim) or gate.shape != out.shape or gate.dtype != out.dtype or gate.stride(1) != 1
            or out.stride(1) != 1):
        raise KernelError("mlstm_out: gate and out must be [T, heads*vdim] of one type with unit inner stride")
    _check(library().arle_mlstm_out(_ptr(num), _ptr(floor), _ptr(gate), _dt(out), gate.stride(0), _ptr(weight), float(eps), _ptr(out),
                                    out.stride(0), T, heads, vdim, _stream()), "mlstm_out")


def ssm_gates(dt_raw, dt_bias, a_log, a, b) -> None:
    """dt = softplus(dt_raw + dt_bias) (no clamp); a = exp(-exp(a_log) * dt); b = dt.  dt_raw float32 [T, heads] (any row
    stride); dt_bias, a_log float32 [heads]; a, b contiguous float32 [T, heads]."""
    T, heads = dt_raw.shape
    if dt_raw.dtype != torch.float32 or dt_raw.stride(1) != 1:
        raise KernelError("ssm_gates: dt_raw must be float32 with unit inner stride")
    for t_ in (dt_bias, a_log):
        if t_.dtype != torch.float32 or t_.numel() != heads:
            raise KernelError("ssm_gates: dt_bias and a_log must be float32 [heads]")
    for t_ in (a, b):
        if t_.dtype != torch.float32 or tuple(t_.shape) != (T, heads) or not t_.is_contiguous():
            raise KernelError("ssm_gates: a and b must be contiguous float32 [T, heads]")
    _check(library().arle_ssm_gates(_ptr(dt_raw), dt_raw.stride(0), _ptr(dt_bias), _ptr(a_log), _ptr(a), _ptr(b), T, heads, _stream()),
           "ssm_gates")


def conv_silu(x, weight, bias, state, conv_offset: int, q_indptr, row_of_token, state_slots, out) -> None:
    """out[t, c] = silu(bias[c] + sum_j weight[c, j] * in[t - (taps - 1) + j, c]) over the tokens of t's row; before the row's
    first token of this step stand the request's last taps - 1 inputs, kept at state[slot, conv_offset + c * (taps - 1) + j]
    (oldest first; zero for a new request) and brought up to date after the convolution.  x, out [T, C] in the activation
    type (views of wider rows are fine); weight float32 [C, taps], bias float32 [C] or None; state float32 [slots, n]."""
    T, C = x.shape
    taps = weight.shape[1]
    R = state_slots.numel()
    if x.stride(1) != 1 or out.stride(1) != 1 or out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("conv_silu: x and out must be [T, C] of one type with unit inner stride")
    if weight.dtype != torch.float32 or weight.shape[0] != C or not weight.is_contiguous() or (
            bias is not None and (bias.dtype != torch.float32 or bias.numel() != C)):
        raise KernelError("conv_silu: weight float32 [C, taps] contiguous, bias float32 [C]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < conv_offset + C * (taps - 1) or state.stride(1) != 1:
        raise KernelError("conv_silu: state must be float32 [slots, n] with room for C * (taps - 1) numbers at conv_offset")
    _i32(q_indptr, "q_indptr"), _i32(row_of_token, "row_of_token"), _i32(state_slots, "state_slots")
    _check(library().arle_conv_silu(_ptr(x), _dt(x), x.stride(0), _ptr(weight), _ptr(bias), _ptr(state), state.stride(0),
                                    int(conv_offset), _ptr(q_indptr), _ptr(row_of_token), _ptr(state_slots), _ptr(out), out.stride(0),
                                    T, R, C, taps, _stream()), "conv_silu")
    if taps > 1:
        add_launches(1)


def gated_group_norm(y, x, skip, vdim: int, z, weight, eps: float, out, parts: int) -> None:
    """out = rms_unit_in_parts((y + skip[head] * x) * silu(z)) * weight: the row of ``inner`` numbers in ``parts`` equal
    parts, each divided by its own root mean square; head = column // vdim.  y float32 [T, inner] contiguous; x, z, out
    [T, inner] in the activation type (views of wider rows are fine); skip float32 [inner / vdim] or None (then x is not
    read); weight float32 [inner]."""
    T, inner = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous() or inner % parts:
        raise KernelError("gated_group_norm: y must be contiguous float32 [T, inner] with inner a multiple of parts")
    for t_ in ((x, z, out) if skip is not None else (z, out)):
        if tuple(t_.shape) != (T, inner) or t_.stride(1) != 1 or t_.dtype != out.dtype:
            raise KernelError("gated_group_norm: x, z and out must be [T, inner] of one type with unit inner stride")
    if weight.dtype != torch.float32 or weight.numel() != inner or (
            skip is not None and (skip.dtype != torch.float32 or skip.numel() * vdim != inner)):
        raise KernelError("gated_group_norm: weight float32 [inner], skip float32 [inner / vdim]")
    _check(library().arle_gated_group_norm(_ptr(y), _ptr(x) if skip is not None else None, _dt(out),
                                           x.stride(0) if skip is not None else 0, _ptr(skip), vdim, _ptr(z), z.stride(0),
                                           _ptr(weight), float(eps), _ptr(out), out.stride(0), T, inner, parts, _stream()),
           "gated_group_norm")


# ------------------------------------------------------------------ routed experts
def moe_select(z, correction, scratch, experts: int, top: int, groups: int, keep: int, scale: float, ids, weights,
               scores: str = "sigmoid", group_score: str = "top2_sum") -> None:
    """Chooses ``top`` experts per token from float32 router sums z [T, >= experts] (any row stride): scores sigmoid(z),
    choice scores with ``correction`` (float32 [experts] or None) added, experts in ``groups`` equal groups of neighbours of
    which only the ``keep`` with the best scores (sum of a group's two largest choice scores) can be chosen; ids int32
    [T, top] in the order chosen, weights float32 [T, top] = sigmoid(z) * scale.  scratch float32 [T, experts + groups].
    ``scores`` "softmax": the scores are softmax(z) over all experts; "softmax_chosen": the sums z themselves decide the
    choice and the weights are the softmax over the chosen sums alone; ``group_score`` "max": a group's score is its
    largest choice score alone."""
    T = z.shape[0]
    if scores not in ("sigmoid", "softmax", "softmax_chosen") or group_score not in ("top2_sum", "max"):
        raise KernelError(f"moe_select: scores {scores!r} / group_score {group_score!r} not known")
    if z.dtype != torch.float32 or z.stride(1) != 1 or z.shape[1] < experts:
        raise KernelError("moe_select: z must be float32 [T, >= experts] with unit inner stride")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != experts):
        raise KernelError("moe_select: correction must be float32 [experts]")
    if scratch.dtype != torch.float32 or scratch.numel() < T * (experts + groups) or not scratch.is_contiguous():
        raise KernelError("moe_select: scratch must be contiguous float32 [T, experts + groups]")
    if (ids.dtype != torch.int32 or weights.dtype != torch.float32 or tuple(ids.shape) != (T, top) or tuple(weights.shape) != (T, top)
            or not ids.is_contiguous() or not weights.is_contiguous()):
        raise KernelError("moe_select: ids int32 [T, top] and weights float32 [T, top], contiguous")
    _check(library().arle_moe_select(_ptr(z), z.stride(0), _ptr(correction), _ptr(scratch), experts, top, groups, keep, float(scale),
                                     int(scores == "softmax") | (int(group_score == "max") << 1) | (int(scores == "softmax_chosen") << 2),
                                     _ptr(ids), _ptr(weights), T,
                                     _stream()), "moe_select")


def moe_plan_size(experts: int, pairs: int) -> int:
    """int32 entries of the plan that ``moe_plan`` writes."""
    lib = library()
    lib.arle_moe_plan_ints.argtypes = [c_int, c_int]
    lib.arle_moe_plan_ints.restype = c_int
    return int(lib.arle_moe_plan_ints(int(experts), int(pairs)))


def moe_plan(ids, experts: int, plan, place_of_pair, row_of_place) -> None:
    """Sorts the pairs (token, choice) of ids [T, top] by expert, on the device: plan (int32, ``moe_plan_size`` entries: the
    experts' runs and the tiles the grouped product runs), place_of_pair int32 [T*top], row_of_place int32 [T*top] (the
    token of the pair at each place)."""
    T, top = ids.shape
    pairs = T * top
    if (ids.dtype != torch.int32 or not ids.is_contiguous() or plan.dtype != torch.int32 or plan.numel() < moe_plan_size(experts, pairs)
            or place_of_pair.dtype != torch.int32 or place_of_pair.numel() < pairs or row_of_place.dtype != torch.int32
            or row_of_place.numel() < pairs):
        raise KernelError("moe_plan: int32 tables of the sizes moe_plan_size gives")
    _check(library().arle_moe_plan(_ptr(ids), pairs, top, experts, _ptr(plan), _ptr(place_of_pair), _ptr(row_of_place), _stream()),
           "moe_plan")


def moe_gemm(x, rows, w, out, plan, experts: int) -> None:
    """out[place] = x[rows[place]] . w[expert of place]^T for every place of the plan (rows None: x is in place order).
    x [*, K], w [experts, N, K] contiguous, out [pairs, N] in x's type; float32 sums, k ascending.  With the fast kernel
    set, bfloat16 operands with rows on 16-byte boundaries run on the tensor cores (many pairs) or as one dot product a
    warp (up to 128 pairs: a decode step)."""
    pairs, N = out.shape
    K = x.shape[1]
    if (w.dim() != 3 or w.shape[0] != experts or w.shape[1] != N or w.shape[2] != K or not w.is_contiguous() or x.stride(1) != 1
            or out.stride(1) != 1 or x.dtype != out.dtype or (x.dtype == torch.bfloat16 and w.dtype != torch.bfloat16)):
        raise KernelError(f"moe_gemm: shapes x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    _i32(rows, "rows"), _i32(plan, "plan")
    _check(library().arle_moe_gemm(_ptr(x), x.stride(0), _ptr(rows), _ptr(w), K, N * K, _ptr(out), out.stride(0), _dt(x), _dt(w),
                                   _ptr(plan), experts, pairs, N, K, int(_KERNEL_SET == "fast"), _stream()), "moe_gemm")


def moe_combine(y, place_of_pair, weights, shared, gate, out) -> None:
    """out[t] = sum_k weights[t, k] * y[place_of_pair[t*top + k]] (k ascending, float32) + sigmoid(gate[t]) * shared[t].
    y [pairs, width]; shared [T, width] or None; gate float32 [T] (any stride) or None (the shared rows are added as
    they are); out [T, width] (unit inner stride)."""
    T, top = weights.shape
    width = out.shape[1]
    if (y.shape[1] != width or y.stride(1) != 1 or out.stride(1) != 1 or y.dtype != out.dtype or weights.dtype != torch.float32
            or not weights.is_contiguous() or out.shape[0] != T):
        raise KernelError("moe_combine: y [pairs, width] and out [T, width] of one type, weights float32 [T, top]")
    if shared is not None and (tuple(shared.shape) != (T, width) or shared.stride(1) != 1 or shared.dtype != out.dtype):
        raise KernelError("moe_combine: shared must be [T, width] in the activation type")
    if gate is not None and (gate.dtype != torch.float32 or gate.numel() != T or gate.dim() != 1):
        raise KernelError("moe_combine: gate must be float32 [T]")
    _i32(place_of_pair, "place_of_pair")
    _check(library().arle_moe_combine(_ptr(y), y.stride(0), _ptr(place_of_pair), _ptr(weights), top, _ptr(shared),
                                      shared.stride(0) if shared is not None else 0, _ptr(gate), gate.stride(0) if gate is not None else 0,
                                      _ptr(out), out.stride(0), _dt(out), T, width, _stream()), "moe_combine")


# ------------------------------------------------------------------ parts of further designs
def clamped_glu(gate_up, out, limit: float, alpha: float) -> None:
    """out[t, i] = g * sigmoid(alpha * g) * (u + 1) with g = min(gate_up[t, 2i], limit) and u = gate_up[t, 2i + 1] clamped to
    [-limit, limit]; float32 arithmetic, rounded once.  ``out`` may be columns of a wider buffer."""
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or not gate_up.is_contiguous() or out.stride(1) != 1 or gate_up.dtype != out.dtype:
        raise KernelError("clamped_glu: gate_up must be contiguous [T, 2I] and out [T, I] of the same type with unit inner stride")
    _check(library().arle_clamped_glu(_ptr(gate_up), _ptr(out), _dt(out), T, I, out.stride(0) if T > 1 else I, float(limit),
                                      float(alpha), _stream()), "clamped_glu")


def branch_norm_add(resid, branch, weight, eps: float, copy) -> None:
    """resid += branch / sqrt(mean(branch^2) + eps) * weight per row, in float32; ``copy`` (or None) gets the new residual
    in its own type.  ``branch`` None: only the copy is written.  resid float32 [T, H] contiguous; branch [T, H] (unit inner
    stride) and copy [T, H] contiguous in the activation type; weight float32 [H]."""
    T, H = resid.shape
    if resid.dtype != torch.float32 or not resid.is_contiguous():
        raise KernelError("branch_norm_add: the residual must be contiguous float32")
    if branch is not None and (tuple(branch.shape) != (T, H) or branch.stride(1) != 1 or weight is None
                               or weight.dtype != torch.float32 or weight.numel() != H):
        raise KernelError("branch_norm_add: branch [T, H] with unit inner stride and weight float32 [H]")
    if copy is not None and (tuple(copy.shape) != (T, H) or not copy.is_contiguous()):
        raise KernelError("branch_norm_add: copy must be contiguous [T, H]")
    if branch is not None and copy is not None and branch.dtype != copy.dtype:
        raise KernelError("branch_norm_add: branch and copy must share a type")
    if branch is None and copy is None:
        return
    _check(library().arle_branch_norm_add(_ptr(resid), _ptr(branch), branch.stride(0) if branch is not None else 0, _ptr(weight),
                                          _ptr(copy), _dt(branch if branch is not None else copy), T, H, float(eps), _stream()),
           "branch_norm_add")


def branch_norm_add_norm(resid, branch, weight, eps: float, next_weight, next_eps: float, out) -> None:
    """resid += branch / sqrt(mean(branch^2) + eps) * weight, then out = resid / sqrt(mean(resid^2) + next_eps) * next_weight,
    per row, in float32, in one kernel: the norm on a sublayer's output and the norm on the next sublayer's input.  resid
    float32 [T, H] contiguous; branch [T, H] (unit inner stride) and out [T, H] contiguous in the activation type; the
    weights float32 [H]."""
    T, H = resid.shape
    if resid.dtype != torch.float32 or not resid.is_contiguous():
        raise KernelError("branch_norm_add_norm: the residual must be contiguous float32")
    if tuple(branch.shape) != (T, H) or branch.stride(1) != 1 or tuple(out.shape) != (T, H) or not out.is_contiguous() or out.dtype != branch.dtype:
        raise KernelError("branch_norm_add_norm: branch [T, H] with unit inner stride, out contiguous [T, H] of the same type")
    for w_ in (weight, next_weight):
        if w_.dtype != torch.float32 or w_.numel() != H:
            raise KernelError("branch_norm_add_norm: weights must be float32 [H]")
    _check(library().arle_branch_norm_add_norm(_ptr(resid), _ptr(branch), branch.stride(0), _ptr(weight), _ptr(next_weight), _ptr(out),
                                               _dt(out), T, H, float(eps), float(next_eps), _stream()), "branch_norm_add_norm")


def rms_rows(x, weight, eps: float, out) -> None:
    """out[t, :] = x[t, :] / sqrt(mean(x[t, :]^2) + eps) * weight (float32 [n] or None) for plain rows: x [T, n] float32 or in
    out's type, out [T, n] in the activation type; both may be columns of wider rows."""
    T, n = x.shape
    if x.stride(1) != 1 or out.stride(1) != 1 or tuple(out.shape) != (T, n) or (x.dtype != out.dtype and x.dtype != torch.float32):
        raise KernelError("rms_rows: x and out [T, n] with unit inner stride, x float32 or of out's type")
    if weight is not None and (weight.dtype != torch.float32 or weight.numel() != n):
        raise KernelError("rms_rows: weight must be float32 [n]")
    _check(library().arle_rms_rows(_ptr(x), _dt(x), x.stride(0), _ptr(weight), _ptr(out), _dt(out), out.stride(0), T, n, float(eps),
                                   _stream()), "rms_rows")


def normed_sum(xs, biases, weights, scales, eps: float, out) -> None:
    """out = sum_m scales[m] * rmsnorm(xs[m] + biases[m]) * weights[m] per row, the norms over the whole row with ``eps``
    inside the root: up to four members [T, H] in out's type (unit inner stride), biases float32 [H] or None each,
    weights float32 [H]; float32 arithmetic, one rounding."""
    n = len(xs)
    T, H = out.shape
    if not 0 < n <= 4 or len(weights) != n or len(scales) != n or (biases is not None and len(biases) != n):
        raise KernelError("normed_sum: one to four members, a weight and a scale each")
    biases = list(biases) if biases is not None else [None] * n
    if out.stride(1) != 1:
        raise KernelError("normed_sum: out must have unit inner stride")
    for x_, b_, w_ in zip(xs, biases, weights):
        if tuple(x_.shape) != (T, H) or x_.stride(1) != 1 or x_.dtype != out.dtype:
            raise KernelError("normed_sum: members must be [T, H] of out's type with unit inner stride")
        if w_.dtype != torch.float32 or w_.numel() != H or (b_ is not None and (b_.dtype != torch.float32 or b_.numel() != H)):
            raise KernelError("normed_sum: weights (and biases) must be float32 [H]")
    ptrs = (ctypes.c_void_p * n)(*[_ptr(x_) for x_ in xs])
    bptrs = (ctypes.c_void_p * n)(*[_ptr(b_) for b_ in biases])
    wptrs = (ctypes.c_void_p * n)(*[_ptr(w_) for w_ in weights])
    strides = (ctypes.c_int * n)(*[x_.stride(0) for x_ in xs])
    sc = (ctypes.c_float * n)(*[float(v) for v in scales])
    _check(library().arle_normed_sum(ptrs, strides, bptrs, wptrs, sc, n, _ptr(out), _dt(out), out.stride(0), T, H, float(eps), _stream()),
           "normed_sum")


def bias_add(x, bias) -> None:
    """x[t, :] += bias (float32 [n]) in place; x [T, n] with unit inner stride (columns of wider rows are fine)."""
    T, n = x.shape
    if x.stride(1) != 1 or bias.dtype != torch.float32 or bias.numel() != n:
        raise KernelError("bias_add: x [T, n] with unit inner stride and bias float32 [n]")
    _check(library().arle_bias_add(_ptr(x), _dt(x), x.stride(0), _ptr(bias), T, n, _stream()), "bias_add")


def attention_prep_post(qkv, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, rotary_dim: int, k_cache, v_cache,
                        nq: int, nkv: int, hd: int, vd: int, page_size: int, norm_first: bool = False) -> None:
    """(``norm_first``: the norm and its weight come before the rotation instead of after it.)  Rotation first, then the per-head norm x / sqrt(mean(x^2) + eps) (times a weight float32 [hd], or none), in place on
    the q heads of qkv [T, nq*hd + nkv*hd + nkv*vd]; the k heads go the same way into k_cache [pages, nkv, page_size, hd]
    and the v heads as they are into v_cache [pages, nkv, page_size, vd] (nkv = 0: the rows hold q only and nothing is
    stored).  ``eps`` None: no norm.  Rotation as in ``attention_prep`` (number i with i + rotary_dim/2)."""
    T = qkv.shape[0]
    if qkv.stride(1) != 1 or qkv.shape[1] < nq * hd + nkv * (hd + vd):
        raise KernelError("attention_prep_post: qkv must be [T, >= nq*hd + nkv*(hd + vd)] with unit inner stride")
    if hd > 256 or rotary_dim % 2 or rotary_dim > hd:
        raise KernelError(f"attention_prep_post: head_dim {hd} / rotary_dim {rotary_dim} not supported")
    for w_ in (q_weight, k_weight):
        if w_ is not None and (w_.dtype != torch.float32 or w_.numel() != hd):
            raise KernelError("attention_prep_post: norm weights must be float32 [head_dim]")
    if nkv > 0:
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
            raise KernelError("attention_prep_post: cache type differs from activation type")
        if (tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or tuple(v_cache.shape[1:]) != (nkv, page_size, vd)
                or not k_cache.is_contiguous() or not v_cache.is_contiguous()):
            raise KernelError(f"attention_prep_post: cache shapes {tuple(k_cache.shape)}, {tuple(v_cache.shape)}")
        _i32(slot_mapping, "slot_mapping")
    _i32(positions, "positions")
    if rotary_dim and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("attention_prep_post: inv_freq must be float32 [rotary_dim / 2]")
    _check(library().arle_attention_prep_post(
        _ptr(qkv), _dt(qkv), qkv.stride(0), _ptr(positions), _ptr(slot_mapping) if nkv else None, _ptr(q_weight), _ptr(k_weight),
        float(eps) if eps is not None else -1.0, _ptr(inv_freq) if rotary_dim else None, int(rotary_dim),
        _ptr(k_cache) if nkv else None, _ptr(v_cache) if nkv else None, nq, nkv, hd, vd, page_size, T, int(bool(norm_first)),
        _stream()), "attention_prep_post")


def causal_conv(x, in_bias, weight, out_bias, act: str, state, conv_offset: int, q_indptr, row_of_token, state_slots, out) -> None:
    """out[t, c] = act(out_bias[c] + sum_j weight[c, j] * in[t - (taps - 1) + j, c]) over the tokens of t's row, where in is
    x + in_bias for the request's tokens and zero before its first; ``act`` "none" or "silu".  The request's last taps - 1
    inputs are kept at state[slot, conv_offset + c * (taps - 1) + j] (oldest first; zero for a new request) and brought up to
    date after the convolution.  x [T, C] in the activation type, out [T, C] in that type or float32 (views of wider rows
    are fine); weight float32 [C, taps]; the biases float32 [C] or None; state float32 [slots, n]."""
    T, C = x.shape
    taps = weight.shape[1]
    R = state_slots.numel()
    if act not in ("none", "silu"):
        raise KernelError(f"causal_conv: act {act!r} (none, silu)")
    if x.stride(1) != 1 or out.stride(1) != 1 or out.shape != x.shape or (out.dtype != x.dtype and out.dtype != torch.float32):
        raise KernelError("causal_conv: x and out must be [T, C] with unit inner stride, out in x's type or float32")
    for b_ in (in_bias, out_bias):
        if b_ is not None and (b_.dtype != torch.float32 or b_.numel() != C):
            raise KernelError("causal_conv: biases must be float32 [C]")
    if weight.dtype != torch.float32 or weight.shape[0] != C or not weight.is_contiguous():
        raise KernelError("causal_conv: weight float32 [C, taps] contiguous")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < conv_offset + C * (taps - 1) or state.stride(1) != 1:
        raise KernelError("causal_conv: state must be float32 [slots, n] with room for C * (taps - 1) numbers at conv_offset")
    _i32(q_indptr, "q_indptr"), _i32(row_of_token, "row_of_token"), _i32(state_slots, "state_slots")
    _check(library().arle_causal_conv(_ptr(x), _dt(x), x.stride(0), _ptr(in_bias), _ptr(weight), _ptr(out_bias), int(act == "silu"),
                                      _ptr(state), state.stride(0), int(conv_offset), _ptr(q_indptr), _ptr(row_of_token),
                                      _ptr(state_slots), _ptr(out), _dt(out), out.stride(0), T, R, C, taps, _stream()), "causal_conv")
    if taps > 1:
        add_launches(1)


def rglru_scan(z, u, y, bias_r, bias_i, lam, y_bias, c_decay: float, state, q_indptr, state_slots, out, blocks: int,
               max_q_len: int) -> None:
    """The real-gated linear recurrent unit over the tokens of every row of the step, from and into state[state_slots[r]]
    (its first ``width`` numbers): r = sigmoid(z_r + bias_r), i = sigmoid(z_i + bias_i), a = exp(-c_decay * r * softplus(lam)),
    S_t = a S_(t-1) + sqrt(1 - a^2) * i * u_t, out_t = S_t * gelu_tanh(y_t + y_bias).  z float32 [T, 2*width] contiguous, per
    token and block of width/blocks channels the recurrence gates' sums, then the input gates'; u [T, width] contiguous
    and y, out [T, width] (views of wider rows are fine) in the activation type; the rest float32 [width]."""
    T, width = u.shape
    R = state_slots.numel()
    if (z.dtype != torch.float32 or tuple(z.shape) != (T, 2 * width) or not z.is_contiguous() or u.dtype != y.dtype
            or not u.is_contiguous() or width % blocks):
        raise KernelError("rglru_scan: z float32 [T, 2*width] and u [T, width] in y's type, contiguous; width a multiple of blocks")
    if tuple(y.shape) != (T, width) or tuple(out.shape) != (T, width) or y.stride(1) != 1 or out.stride(1) != 1 or y.dtype != out.dtype:
        raise KernelError("rglru_scan: y and out must be [T, width] of one type with unit inner stride")
    for t_ in (bias_r, bias_i, lam) + ((y_bias,) if y_bias is not None else ()):
        if t_.dtype != torch.float32 or t_.numel() != width or not t_.is_contiguous():
            raise KernelError("rglru_scan: biases and lam must be contiguous float32 [width]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < width or state.stride(1) != 1:
        raise KernelError("rglru_scan: state must be float32 [slots, >= width]")
    _i32(q_indptr, "q_indptr"), _i32(state_slots, "state_slots")
    if q_indptr.numel() != R + 1:
        raise KernelError("rglru_scan: q_indptr must have one entry more than state_slots")
    _check(library().arle_rglru_scan(_ptr(z), _ptr(u), _ptr(y), _dt(y), y.stride(0), _ptr(bias_r), _ptr(bias_i), _ptr(lam), _ptr(y_bias),
                                     float(c_decay), _ptr(state), state.stride(0), _ptr(q_indptr), _ptr(state_slots), _ptr(out),
                                     out.stride(0), R, width, blocks, max(int(max_q_len), 1), _stream()), "rglru_scan")


def delta_gates(pre, a_log, dt_bias, beta, decay) -> None:
    """beta = sigmoid(pre[:, :H]); decay = exp(-exp(a_log) * softplus(pre[:, H:] + dt_bias)); pre float32 [T, 2H] (any row
    stride); a_log, dt_bias float32 [H]; beta, decay float32 [T, H] contiguous."""
    T, H = beta.shape
    if pre.dtype != torch.float32 or pre.shape[0] != T or pre.shape[1] < 2 * H or pre.stride(1) != 1:
        raise KernelError("delta_gates: pre must be float32 [T, >= 2H] with unit inner stride")
    for t_ in (a_log, dt_bias):
        if t_.dtype != torch.float32 or t_.numel() != H:
            raise KernelError("delta_gates: a_log and dt_bias must be float32 [H]")
    for t_ in (beta, decay):
        if t_.dtype != torch.float32 or tuple(t_.shape) != (T, H) or not t_.is_contiguous():
            raise KernelError("delta_gates: beta and decay must be contiguous float32 [T, H]")
    _check(library().arle_delta_gates(_ptr(pre), pre.stride(0), _ptr(a_log), _ptr(dt_bias), _ptr(beta), _ptr(decay), T, H, _stream()),
           "delta_gates")


def delta_scan(q, k, v, beta, decay, state, q_indptr, state_slots, out, heads: int, kq_heads: int, dim: int, vdim: int,
               q_scale: float, unit_eps: float) -> None:
    """The gated delta rule over the tokens of every row of the step, from and into state[state_slots[r]]: with q and k brought
    to unit length per head (x / sqrt(sum x^2 + unit_eps); q also times q_scale), S <- decay_t S; u = beta_t (v_t - S^T k_t);
    S <- S + k_t u^T; o_t = S^T q_t.  q, k [T, kq_heads*dim] (head h reads head h // (heads / kq_heads)), v [T, heads*vdim], in
    the activation type (views of wider rows are fine); beta, decay float32 [T, heads]; state float32 [slots, n] whose first
    heads * vdim * dim numbers are the memories, a head's transposed ([heads][vdim][dim]); out float32 [T, heads, vdim]."""
    T = v.shape[0]
    R = state_slots.numel()
    if (q.shape != (T, kq_heads * dim) or k.shape != q.shape or v.shape != (T, heads * vdim) or q.dtype != k.dtype
            or q.dtype != v.dtype or q.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1):
        raise KernelError("delta_scan: q, k [T, kq_heads*dim] and v [T, heads*vdim] of one type with unit inner stride")
    for t_, n_ in ((beta, "beta"), (decay, "decay")):
        if t_.dtype != torch.float32 or tuple(t_.shape) != (T, heads) or not t_.is_contiguous():
            raise KernelError(f"delta_scan: {n_} must be contiguous float32 [T, heads]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < heads * vdim * dim or state.stride(1) != 1:
        raise KernelError(f"delta_scan: state {tuple(state.shape)} must be float32 [slots, >= {heads * vdim * dim}]")
    if out.dtype != torch.float32 or tuple(out.shape) != (T, heads, vdim) or not out.is_contiguous():
        raise KernelError("delta_scan: out must be contiguous float32 [T, heads, vdim]")
    _i32(q_indptr, "q_indptr"), _i32(state_slots, "state_slots")
    if q_indptr.numel() != R + 1:
        raise KernelError("delta_scan: q_indptr must have one entry more than state_slots")
    _check(library().arle_delta_scan(_ptr(q), _ptr(k), _ptr(v), _dt(q), q.stride(0), k.stride(0), v.stride(0), _ptr(beta), _ptr(decay),
                                     _ptr(state), state.stride(0), _ptr(q_indptr), _ptr(state_slots), _ptr(out), T, R, heads, kq_heads,
                                     dim, vdim, float(q_scale), float(unit_eps), _stream()), "delta_scan")
