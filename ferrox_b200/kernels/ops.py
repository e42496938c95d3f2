"""Thin Python entry to the kernels: torch tensors in, pointers out.

Each function checks what the C side cannot (device, contiguity, dtype), passes
pointers, sizes and the current CUDA stream to ``libferrox_b200.so`` and raises
:class:`KernelError` on a non-zero status.  Nothing here computes: there is no
torch fallback, and a CPU tensor is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_long, c_ulonglong, c_void_p
from typing import Optional

import torch

from . import lib as _libmod

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

_ERRORS = {
    -1: "combination of element types not built",
    -2: "a size outside what the kernel handles",
    -3: "pointer or stride not aligned as the kernel requires",
    -4: "a bounded wait inside a kernel ran out",
    -5: "the request needs more scratch than the library's fixed array holds",
}


class KernelError(RuntimeError):
    pass


_P, _I, _L, _F = c_void_p, c_int, c_long, c_float
_SIGNATURES = {
    "fx_set_pdl": [_I],
    "fx_set_scan_lanes": [_I],
    "fx_gemm": [_P, _I, _L, _P, _P, _I, _L, _P, _I, _P, _I, _L, _I, _I, _I, _I, _P, _I, _L, _P],
    "fx_embed": [_P, _I, _P, _P, _I, _I, _I, _P, _F, _P],
    "fx_scaled_add_norm": [_P, _P, _F, _P, _I, _F, _P, _I, _I, _I, _P],
    "fx_rmsnorm": [_P, _P, _P, _I, _F, _P, _I, _I, _I, _P],
    "fx_silu_mul": [_P, _L, _P, _L, _I, _P, _I, _I, _P],
    "fx_rope_kv_write": [_P, _I, _L, _P, _P, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "fx_rope_table": [_P, _P, _I, _I, _P, _F, _P],
    "fx_gemm_tc": [_P, _L, _P, _L, _L, _I, _P, _I, _P, _I, _L, _I, _I, _I, _I, _I, _I, _F, _F, _P, _I, _P, _P],
    "fx_gemm_tc_swap": [_P, _L, _P, _L, _L, _I, _P, _I, _P, _I, _L, _I, _I, _I, _I, _I, _I, _F, _F, _P, _I, _I, _I, _I, _P, _P,
                        _P],
    "fx_gemm_tc2": [_P, _L, _P, _L, _I, _P, _I, _P, _I, _L, _I, _I, _I, _I, _I, _I, _F, _F, _P, _P],
    "fx_gather_rows": [_P, _L, _P, _P, _L, _I, _I, _I, _P],
    "fx_gather_rows_scaled": [_P, _L, _P, _P, _P, _I, _P, _L, _I, _I, _I, _P],
    "fx_paged_attention_ex": [_P, _L, _L, _P, _P, _L, _L, _I, _P, _I, _I, _P, _P, _P, _P, _L, _L, _I, _I, _I, _I, _I, _I, _F,
                              _F, _P, _I, _P, _I, _P],
    "fx_general_attention_ok": [_I, _I, _I],
    "fx_general_attention": [_P, _L, _L, _P, _P, _L, _L, _P, _P, _I, _I, _P, _P, _P, _P, _I, _P, _L, _L, _I, _I, _I, _I, _I,
                             _F, _P, _I, _P, _P, _I, _F, _P, _I, _P],
    "fx_qk_norm_store": [_P, _I, _L, _P, _P, _P, _P, _P, _I, _F, _F, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _F,
                         _P],
    "fx_latent_prep": [_P, _L, _P, _L, _I, _P, _P, _P, _P, _I, _F, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P,
                       _I, _P],
    "fx_rmsnorm_rows": [_P, _I, _L, _P, _I, _F, _P, _I, _L, _I, _I, _P],
    "fx_heads_to_tokens": [_P, _L, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P],
    "fx_route_small": [_P, _L, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P, _F, _F, _P],
    "fx_route": [_P, _L, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _P, _F, _F, _P],
    "fx_route_fused": [_P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _P, _L, _P, _P, _P, _P, _P, _P, _I, _P, _L, _P, _F, _F, _P],
    "fx_moe_combine": [_P, _P, _I, _P, _P, _I, _P, _P, _L, _I, _I, _P],
    "fx_moe_combine_norm": [_P, _P, _I, _P, _P, _I, _P, _P, _L, _I, _I, _P, _I, _F, _P, _P],
    "fx_residual_add": [_P, _P, _I, _L, _P],
    "fx_paged_attention": [_P, _L, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _F, _F, _P],
    "fx_glu_mul": [_P, _L, _P, _L, _I, _P, _I, _I, _I, _F, _F, _P],
    "fx_layernorm": [_P, _P, _P, _I, _P, _I, _F, _P, _I, _I, _I, _P],
    "fx_layernorm_residual": [_P, _P, _I, _F, _P, _I, _F, _P, _I, _F, _P, _I, _F, _P, _I, _I, _I, _P],
    "fx_scale": [_P, _L, _F, _P],
    "fx_delta_prep": [_P, _I, _L, _P, _I, _I, _P, _P, _L, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "fx_conv_tail_update": [_P, _I, _L, _I, _I, _P, _P, _P, _I, _I, _P],
    "fx_state_scan": [_P, _L, _P, _L, _P, _L, _I, _I, _P, _L, _P, _P, _P, _L, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "fx_gated_group_norm": [_P, _P, _I, _L, _P, _I, _F, _I, _P, _I, _I, _I, _I, _L, _P],
    "fx_general_delta_prep": [_P, _L, _P, _L, _P, _L, _P, _I, _P, _I, _P, _I, _F, _P, _P, _P, _I, _I, _I, _I, _P],
    "fx_general_delta_scan": [_P, _L, _P, _L, _P, _L, _P, _P, _P, _P, _P, _L, _P, _P, _I, _I, _I, _I, _P],
    "fx_input_conv": [_P, _I, _L, _P, _I, _I, _P, _P, _P, _P, _L, _I, _I, _I, _I, _P],
    "fx_mlstm_column_blocks": [_I, _I],
    "fx_mlstm_scan": [_P, _L, _P, _L, _P, _L, _P, _L, _P, _P, _I, _F, _F, _P, _P, _P, _P, _L, _P, _P, _I, _I, _I, _I, _I, _I,
                      _P],
    "fx_conv_rotary_store": [_P, _I, _L, _P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                             _I, _I, _I, _I, _P, _P],
    "fx_diff_combine": [_P, _L, _P, _L, _I, _I, _I, _I, _I, _F, _F, _F, _P],
    "fx_embed_pos": [_P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _P, _P],
    "fx_softcap": [_P, _L, _F, _P],
    "fx_relu_square": [_P, _I, _L, _I, _I, _P],
    "fx_prefill_attention": [_P, _L, _P, _P, _P, _I, _I, _P, _I, _P, _P, _L, _I, _I, _I, _I, _F, _F, _P],
    "fx_prefill_attention_tc": [_P, _L, _I, _P, _P, _I, _P, _I, _I, _P, _I, _P, _P, _L, _I, _I, _I, _I, _F, _P, _P, _P,
                                _P, _I, _P],
    "fx_router_topk": [_P, _L, _I, _I, _I, _I, _P, _P, _P, _F, _F, _P],
    "fx_moe_align": [_P, _I, _I, _I, _P, _P, _P, _P, _P, _I, _P],
    "fx_gemm_slab_ok": [_I, _I, _I],
    "fx_gemm_slab": [_P, _L, _P, _L, _P, _I, _P, _I, _L, _I, _I, _I, _I, _P, _P],
    "fx_gemm_skinny": [_P, _L, _P, _P, _L, _L, _P, _I, _P, _I, _L, _I, _I, _I, _I, _I, _I, _F, _F, _P, _P, _I, _I, _I, _P],
    "fx_decode_attention": [_P, _L, _P, _P, _I, _I, _P, _I, _I, _P, _P, _P, _P, _L, _P, _P, _I, _I, _I, _I, _I, _F, _I,
                            _I, _P, _P, _I, _I, _I, _P, _F, _P],
    "fx_argmax": [_P, _L, _I, _I, _P, _P],
    "fx_repetition_penalty": [_P, _L, _I, _I, _P, _P, _P, _P],
    "fx_sample": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P],
    "fx_sample_or": [_P, _L, _P, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P],
    "fx_random_normal": [_P, _I, _L, c_ulonglong, c_double, c_double, _P],
}

_fn = {}

# kernels launched by one call of an entry point (fx_moe_align: count, scan, place)
_KERNELS = {"fx_moe_align": 3, "fx_route": 2, "fx_decode_attention": 2}   # (a split-K product adds a second kernel; not counted)
_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far by this process."""
    return _launches


def count_launches(n: int) -> None:
    """Account for kernels launched outside :func:`call` (a CUDA graph's replay)."""
    global _launches
    _launches += n


def _get(name: str):
    f = _fn.get(name)
    if f is None:
        lib = _libmod.load()
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[name]
        f.restype = c_int
        _fn[name] = f
    return f


def register_signature(name: str, argtypes) -> None:
    """Lets further source files of the library declare their entry points."""
    _SIGNATURES[name] = list(argtypes)


def call(name: str, *args) -> None:
    global _launches
    _launches += _KERNELS.get(name, 1)
    if _trace is not None:
        return _call_traced(name, args)
    rc = _get(name)(*args)
    if rc != 0:
        if rc > 0:
            raise KernelError(f"{name}: CUDA error {rc} at launch ({torch.cuda.get_device_name()})")
        raise KernelError(f"{name}: refused: {_ERRORS.get(rc, rc)}")


# ---- tracing: device time per class of kernel, behind a switch -------------------------------------------
# The reference prints phase rates only (crates/ferrox-cli/src/run.rs:680-695); with the switch on, every entry
# point's launches are bracketed by CUDA events on their own stream and summed by (scope, entry point), where the
# scope is what the parts announce with :class:`trace_scope` (mixer, feed-forward, norm, head ...).  Launches then
# run without programmatic dependent launch, so that a kernel's time is its own; the engine leaves CUDA graphs off.
_trace = None          # None: off; else {key: [n_calls, [(start event, end event), ...]]}
_trace_scope = []


def trace_enabled() -> bool:
    return _trace is not None


def trace_start() -> None:
    global _trace
    _trace = {}
    _get("fx_set_pdl")(0)


def trace_stop() -> dict:
    """Ends tracing; returns {"scope:entry point": (launches, milliseconds on the device)}."""
    global _trace
    t, _trace = _trace or {}, None
    _get("fx_set_pdl")(1)
    torch.cuda.synchronize()
    return {k: (n, sum(a.elapsed_time(b) for a, b in evs)) for k, (n, evs) in t.items()}


class trace_scope:
    """Names the part whose kernels follow (no cost while tracing is off)."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _trace is not None:
            _trace_scope.append(self.name)
        return self

    def __exit__(self, *exc):
        if _trace is not None and _trace_scope:
            _trace_scope.pop()
        return False


def _call_traced(name: str, args) -> None:
    stream = torch.cuda.ExternalStream(args[-1]) if args and isinstance(args[-1], int) and args[-1] else torch.cuda.current_stream()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    rc = _get(name)(*args)
    b.record(stream)
    if rc != 0:
        raise KernelError(f"{name}: status {rc}")
    key = f"{_trace_scope[-1] if _trace_scope else '-'}:{name}"
    rec = _trace.setdefault(key, [0, []])
    rec[0] += _KERNELS.get(name, 1)
    rec[1].append((a, b))


_scoped_stream = None
_sm_count = 0


def sm_count() -> int:
    """Streaming multiprocessors of the current device, asked once; launch shapes and the choices between kernels are
    functions of it.  Without a device (the choices are also tested on the CPU): the B200's 148."""
    global _sm_count
    if _sm_count == 0:
        if not torch.cuda.is_available():
            return 148
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def stream_ptr() -> int:
    """The stream kernels go to when none is named: the one a step has announced, else torch's current stream."""
    if _scoped_stream is not None:
        return _scoped_stream
    return torch.cuda.current_stream().cuda_stream


class stream_scope:
    """While a step runs, its stream is known: asking torch for the current stream costs more than a launch."""

    def __init__(self, ptr: int):
        self.ptr = ptr

    def __enter__(self):
        global _scoped_stream
        self.prev, _scoped_stream = _scoped_stream, self.ptr
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self.prev
        return False


def code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not handled by the kernels") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels take CUDA tensors only (there is no CPU path)")
    return t.data_ptr()


def _rows(t: torch.Tensor) -> int:
    """Row stride of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"expected a 2-D tensor with contiguous rows, found shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


# ---------------------------------------------------------------------------
def gemm(a, w, out, *, bias=None, accumulate=False, a_rows=None, group_offsets=None, stream=None):
    """out[M,N] (+)= a[M,K] . w[N,K]^T (+ bias).  With ``group_offsets`` ([G+1],
    int32) ``w`` is [G,N,K] and rows off[g]..off[g+1] use matrix g; ``a_rows``
    gathers rows of ``a``."""
    M, N = out.shape
    if group_offsets is not None:
        G, Nw, K = w.shape
        wstride = w.stride(0)
        ldw = w.stride(1)
        if w.stride(2) != 1:
            raise KernelError("grouped weights must have contiguous rows")
    else:
        G, wstride = 1, 0
        Nw, K = w.shape
        ldw = _rows(w)
    if Nw != N or a.shape[1] != K or (a_rows is None and a.shape[0] != M):
        raise KernelError(f"gemm shapes do not agree: a {tuple(a.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call(
        "fx_gemm", _ptr(a), code(a), _rows(a), _ptr(a_rows), _ptr(w), code(w), ldw,
        _ptr(bias), code(bias) if bias is not None else 0, _ptr(out), code(out), _rows(out), int(accumulate),
        M, N, K, _ptr(group_offsets), G, wstride, stream if stream is not None else stream_ptr(),
    )
    return out


def embed(table, ids, out, status=None, stream=None, scale=1.0):
    """out[t] = table[ids[t]] * scale in 32 bits."""
    T = ids.numel()
    call("fx_embed", _ptr(table), code(table), _ptr(ids), _ptr(out), T, table.shape[1], table.shape[0], _ptr(status),
         float(scale), stream if stream is not None else stream_ptr())
    return out


def scaled_add_norm(h, y, scale, norm=None, stream=None):
    """h += scale * y over the 32-bit rows of the residual stream; ``norm`` = (weight, eps, out): also out = h /
    sqrt(mean(h^2) + eps) * weight on the new rows, in the same kernel.  Returns ``out`` (None without a norm)."""
    if h.dtype != torch.float32 or y.dtype != torch.float32 or h.shape != y.shape or not (h.is_contiguous() and y.is_contiguous()):
        raise KernelError("scaled_add_norm: two contiguous 32-bit tensors of one shape")
    w, eps, out = norm if norm is not None else (None, 0.0, None)
    call("fx_scaled_add_norm", _ptr(h), _ptr(y), float(scale), _ptr(w), code(w) if w is not None else 0, float(eps),
         _ptr(out), code(out) if out is not None else 0, h.shape[0], h.shape[1],
         stream if stream is not None else stream_ptr())
    return out


def rmsnorm(x, weight, eps, out, rows=None, stream=None):
    if x.dtype != torch.float32:
        raise KernelError("rmsnorm reads the 32-bit residual stream")
    n = out.shape[0]
    call("fx_rmsnorm", _ptr(x), _ptr(rows), _ptr(weight), code(weight), float(eps), _ptr(out), code(out), n, x.shape[1],
         stream if stream is not None else stream_ptr())
    return out


GATE_ACTIVATIONS = {"silu": 0, "relu": 1, "clamped_swish": 2}   # what a gated feed-forward passes its gate through


UNARY_ACTIVATIONS = {"relu_square": 1}     # what a plain product's result may pass through in the kernel's epilogue


def unary_code(activation) -> int:
    """The product kernels' code of an activation on their result (0 for None)."""
    if activation is None:
        return 0
    try:
        return UNARY_ACTIVATIONS[activation]
    except (KeyError, TypeError):
        raise KernelError(f"activation {activation!r}: the product kernels know {', '.join(UNARY_ACTIVATIONS)}") from None


def _gated_or_unary(gated, unary):
    """The kernels' ``gated`` argument: the gate's code, or minus the code of a plain product's activation."""
    u = unary_code(unary)
    if u and gated:
        raise KernelError("a gated product takes no second activation")
    return -u if u else gated


def gate_code(activation) -> int:
    """``activation``: a name, or (name, limit, alpha) for the clamped unit
    min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + 1)."""
    name = activation[0] if isinstance(activation, tuple) else activation
    try:
        c = GATE_ACTIVATIONS[name]
    except (KeyError, TypeError):
        raise KernelError(f"gate activation {activation!r}: the kernels know {', '.join(GATE_ACTIVATIONS)}") from None
    if (c == 2) != isinstance(activation, tuple) or (c == 2 and len(activation) != 3):
        raise KernelError("the clamped gate activation is given as (name, limit, alpha), the others by name")
    return c


def _gate_args(gated):
    """The kernels' (gated, act_limit, act_alpha): ``gated`` is 0 / False (plain), 1 / True (SiLU gate), 2 (ReLU gate)
    or (3, limit, alpha) (the clamped unit)."""
    if isinstance(gated, tuple):
        return int(gated[0]), float(gated[1]), float(gated[2])
    return int(gated), 0.0, 0.0


def gated_arg(activation):
    """What the product kernels take as ``gated`` for a gate activation (see :func:`gate_code`)."""
    c = gate_code(activation)
    return (3, float(activation[1]), float(activation[2])) if c == 2 else 1 + c


def silu_mul(gu, out, stream=None, activation="silu"):
    """out = act(gate) * up over rows of [gate | up]."""
    rows, n = out.shape
    if gu.shape[1] != 2 * n:
        raise KernelError("silu_mul expects [gate | up] rows of twice the output width")
    lim, alpha = (float(activation[1]), float(activation[2])) if isinstance(activation, tuple) else (0.0, 0.0)
    call("fx_glu_mul", _ptr(gu), _rows(gu), _ptr(out), _rows(out), code(gu), None, rows, n, gate_code(activation),
         lim, alpha, stream if stream is not None else stream_ptr())
    return out


def layernorm(x, weight, eps, out, rows=None, stream=None, bias=None):
    """out = (x - mean) / sqrt(var + eps) * weight (+ bias) over rows of the 32-bit stream ``x`` (``out`` may be
    ``x``)."""
    if x.dtype != torch.float32:
        raise KernelError("layernorm reads the 32-bit residual stream")
    call("fx_layernorm", _ptr(x), _ptr(rows), _ptr(weight), code(weight), _ptr(bias), code(bias) if bias is not None else 0,
         float(eps), _ptr(out), code(out), out.shape[0], x.shape[1], stream if stream is not None else stream_ptr())
    return out


def layernorm_residual(h, y, weight, eps, *, scale=1.0, y2=None, scale2=1.0, then=None, stream=None):
    """h += ln(scale * y + scale2 * y2) * weight, the norm over whole rows.  ``then`` = (weight, eps, out): also
    out = ln(new h) * weight, in the same kernel."""
    T, H = h.shape
    if h.dtype != torch.float32 or y.shape != h.shape or (y2 is not None and y2.shape != h.shape):
        raise KernelError("layernorm_residual: the stream is 32-bit and the sublayer's output has its shape")
    for t in (y, y2):
        if t is not None and not t.is_contiguous():
            raise KernelError("layernorm_residual takes contiguous rows")
    wn, en, out = then if then is not None else (None, 0.0, None)
    call("fx_layernorm_residual", _ptr(h), _ptr(y), code(y), float(scale), _ptr(y2), code(y2) if y2 is not None else 0,
         float(scale2), _ptr(weight), code(weight), float(eps), _ptr(wn), code(wn) if wn is not None else 0, float(en),
         _ptr(out), code(out) if out is not None else 0, T, H, stream if stream is not None else stream_ptr())
    return out


def scale_(x, factor, stream=None):
    """x *= factor (32-bit, in place)."""
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_ takes a contiguous 32-bit tensor")
    call("fx_scale", _ptr(x), x.numel(), float(factor), stream if stream is not None else stream_ptr())
    return x


def delta_prep(proj, conv_w, taps, tail, ba, a_log, dt_bias, token_seq, seq_slot, out, beta, g, G, D, H, V, stream=None,
               update_tail=False):
    """What the gated delta rule needs before its recurrence, from rows ``proj`` = [q | k | v | ...] as projected:
    short causal convolution (``conv_w`` [channels, taps], the inputs before the step from ``tail`` [slots, taps-1,
    channels]) and SiLU, q and k to unit length per head (q also times D^-1/2), into ``out`` [T, channels] 32-bit;
    beta = sigmoid(b) and g = exp(-exp(A_log) softplus(a + dt_bias)) from ``ba`` = [b | a] 32-bit rows.
    ``update_tail``: only when every entry of the step brings exactly one token; the kernel then also moves the
    tail on, and :func:`conv_tail_update` is not needed."""
    T = proj.shape[0]
    call("fx_delta_prep", _ptr(proj), code(proj), _rows(proj), _ptr(conv_w), code(conv_w), int(taps), _ptr(tail), _ptr(ba),
         _rows(ba), _ptr(a_log), _ptr(dt_bias), _ptr(token_seq), _ptr(seq_slot), _ptr(out), _ptr(beta), _ptr(g), T, G, D, H, V,
         int(update_tail), stream if stream is not None else stream_ptr())


def conv_tail_update(proj, channels, taps, tail, token_seq, seq_slot, n_entries, stream=None):
    """The last ``taps - 1`` inputs of every entry of the step become its request's convolution tail."""
    call("fx_conv_tail_update", _ptr(proj), code(proj), _rows(proj), int(channels), int(taps), _ptr(tail), _ptr(token_seq),
         _ptr(seq_slot), proj.shape[0], int(n_entries), stream if stream is not None else stream_ptr())


def state_scan(q, k, v, g, g_ld, beta, state, out, token_seq, seq_slot, n_entries, H, G, D, V, silu_on_load=False,
               stream=None):
    """The recurrence of a mixer with a matrix state per head, over every entry's tokens in order:
    ``beta`` None:  S = g S + k v^T;  else  S = g S; u = beta (v - S^T k); S += k u^T;  then out = S^T q.
    ``q``, ``k`` [T, G*D] and ``v`` [T, H*V] are row views (one element type); ``g`` is [T, H] with row stride
    ``g_ld`` (0: one decay per head); ``state`` [slots, H, V, D] and ``out`` [T, H*V] are 32-bit."""
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise KernelError("state_scan: q, k and v share one element type")
    if state.dtype != torch.float32 or out.dtype != torch.float32 or g.dtype != torch.float32:
        raise KernelError("state_scan: state, decays and read-out are 32-bit")
    T = q.shape[0]
    call("fx_state_scan", _ptr(q), _rows(q), _ptr(k), _rows(k), _ptr(v), _rows(v), code(q), int(silu_on_load), _ptr(g),
         int(g_ld), _ptr(beta), _ptr(state), _ptr(out), _rows(out), _ptr(token_seq), _ptr(seq_slot), T, int(n_entries),
         H, G, D, V, stream if stream is not None else stream_ptr())
    return out


GROUP_NORM_GATES = {"silu": 0, "sigmoid": 1}


def gated_group_norm(x, gate, weight, eps, gate_activation, out, groups, width, stream=None):
    """out[t, g, :] = x[t, g, :] / sqrt(mean(x[t, g, :]^2) + eps) * weight * act(gate[t, g, :]); ``x`` 32-bit
    [T, groups*width], ``gate`` a row view of the same width, ``weight`` [width] (shared by the groups) or
    [groups*width] (a weight for every element of the row)."""
    if weight.numel() not in (width, groups * width):
        raise KernelError("gated_group_norm: a weight per group element, or one for every element of the row")
    call("fx_gated_group_norm", _ptr(x), _ptr(gate), code(gate), _rows(gate), _ptr(weight), code(weight), float(eps),
         GROUP_NORM_GATES[gate_activation], _ptr(out), code(out), x.shape[0], int(groups), int(width),
         int(width) if weight.numel() != width else 0, stream if stream is not None else stream_ptr())
    return out


def general_delta_prep(k, a_pre, w1_out, w2, w0, a_bias, rate, u, au, w, H, D, stream=None):
    """What the generalized delta rule needs before its recurrence, per (token, head), from 32-bit row views ``k``
    [T, H*D], ``a_pre`` [T, H*D] and ``w1_out`` [T, rank]: the unit key u = k / sqrt(sum k^2 + 1e-6), a u with
    a = sigmoid(a_pre + a_bias), and the decay w = exp(-rate sigmoid(w2 . tanh(w1_out) + w0)); ``u``, ``au``, ``w``
    contiguous 32-bit [T, H*D]."""
    for t in (k, a_pre, w1_out, u, au, w):
        if t.dtype != torch.float32:
            raise KernelError("general_delta_prep: what enters the recurrence is 32-bit")
    T, rank = k.shape[0], w1_out.shape[1]
    call("fx_general_delta_prep", _ptr(k), _rows(k), _ptr(a_pre), _rows(a_pre), _ptr(w1_out), _rows(w1_out), _ptr(w2),
         code(w2), _ptr(w0), code(w0), _ptr(a_bias), code(a_bias), float(rate), _ptr(u), _ptr(au), _ptr(w), T, int(H),
         int(D), int(rank), stream if stream is not None else stream_ptr())


def general_delta_scan(r, k, v, u, au, w, state, out, token_seq, seq_slot, n_entries, H, D, stream=None):
    """The generalized delta rule over every entry's tokens in order: S = diag(w) S - (a u)(u^T S) + k v^T,
    out = S^T r.  ``r``, ``k``, ``v`` 32-bit row views [T, H*D]; ``u``, ``au``, ``w`` contiguous [T, H*D]; ``state``
    [slots, H, D, D] (column by column) and ``out`` [T, H*D] 32-bit."""
    for t in (r, k, v, u, au, w, state, out):
        if t.dtype != torch.float32:
            raise KernelError("general_delta_scan: the recurrence is 32-bit")
    call("fx_general_delta_scan", _ptr(r), _rows(r), _ptr(k), _rows(k), _ptr(v), _rows(v), _ptr(u), _ptr(au), _ptr(w),
         _ptr(state), _ptr(out), _rows(out), _ptr(token_seq), _ptr(seq_slot), r.shape[0], int(n_entries), int(H), int(D),
         stream if stream is not None else stream_ptr())
    return out


def mlstm_column_blocks(head_dim: int, value_dim: int) -> int:
    """Blocks of value columns :func:`mlstm_scan` shares a head's state out over: the copies of the normaliser and of
    the running maximum that the state keeps.  A function of the two sizes alone, stated here as the kernel's
    launcher states it (128 threads a block; 4 lanes a column, doubled while a lane would hold more than 16 rows, rows
    counted in runs of four), so that a cache can be laid out without the library; the launcher refuses a state laid
    out otherwise."""
    D, V = int(head_dim), int(value_dim)
    if not (0 < D <= 512 and V > 0):
        raise KernelError(f"mlstm: heads of {head_dim} x {value_dim} are outside what the recurrence kernel holds")
    lanes = 4
    while lanes < 32 and -(-D // (4 * lanes)) * 4 > 16:
        lanes *= 2
    cols = 128 // lanes
    return -(-V // cols)


def mlstm_scan(q, k, v, gates, i_bias, f_bias, cap, q_scale, matrix, normalizer, log_max, out, token_seq, seq_slot,
               n_entries, H, D, V, stream=None):
    """The mLSTM recurrence over every entry's tokens in order (see csrc/mlstm.cu).  ``q``, ``k`` [T, H*D], ``v``
    [T, H*V] and ``gates`` [T, >= 2H] (input gates' then forget gates' pre-activations) are 32-bit row views;
    ``matrix`` [slots, H, V, D], ``normalizer`` [slots, H, Z, D] and ``log_max`` [slots, H, Z] the requests' states
    (Z = :func:`mlstm_column_blocks`); ``out`` [T, H*V] 32-bit."""
    for t in (q, k, v, gates, out, matrix, normalizer, log_max):
        if t.dtype != torch.float32:
            raise KernelError("mlstm_scan: 32-bit rows and states")
    if i_bias.dtype != f_bias.dtype:
        raise KernelError("mlstm_scan: both gate biases of one element type")
    call("fx_mlstm_scan", _ptr(q), _rows(q), _ptr(k), _rows(k), _ptr(v), _rows(v), _ptr(gates), _rows(gates), _ptr(i_bias),
         _ptr(f_bias), code(i_bias), float(cap), float(q_scale), _ptr(matrix), _ptr(normalizer), _ptr(log_max), _ptr(out),
         _rows(out), _ptr(token_seq), _ptr(seq_slot), q.shape[0], int(n_entries), H, D, V, int(normalizer.shape[2]),
         stream if stream is not None else stream_ptr())
    return out


def conv_rotary_store(proj, weight, taps, tail, positions, token_seq, seq_slot, cos_sin, rot_dims, pairing, q_out,
                      k_pages, v_pages, block_table, page_size, n_q_heads, n_k_heads, head_dim, n_v_heads, value_dim,
                      write_cache=True, update_tail=False, status=None, stream=None):
    """Rows of [q heads | k heads | v heads] as projected: a short causal convolution on every channel (``weight``
    [channels, taps], nothing added; the inputs before the step from ``tail`` [slots, taps - 1, channels] 32-bit),
    the first ``rot_dims`` elements of every q and k head turned by ``cos_sin`` [T, rot_dims / 2, 2] (None: no
    rotation), q into ``q_out`` [T, n_q_heads * head_dim], k and v into their pages ([pages, n_k_heads, page,
    head_dim], [pages, n_v_heads, page, value_dim]).  ``update_tail``: only when every entry brings exactly one
    token; the kernel then moves the tail on (:func:`conv_tail_update` on ``proj`` otherwise)."""
    if q_out.dtype != proj.dtype or k_pages.dtype != proj.dtype or v_pages.dtype != proj.dtype:
        raise KernelError("conv_rotary_store: rows, queries and pages of one element type")
    call("fx_conv_rotary_store", _ptr(proj), code(proj), _rows(proj), _ptr(weight), code(weight), int(taps), _ptr(tail),
         _ptr(positions), _ptr(token_seq), _ptr(seq_slot), _ptr(cos_sin), int(rot_dims if cos_sin is not None else 0),
         int(pairing), _ptr(q_out), _rows(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
         page_size, proj.shape[0], n_q_heads, n_k_heads, head_dim, n_v_heads, value_dim, int(write_cache),
         int(update_tail), _ptr(status), stream if stream is not None else stream_ptr())
    return q_out


def diff_combine(attn, out, n_heads, group, value_dim, lam, eps, post, stream=None):
    """out[t, h] = rms(a1 - lam * a2) * post per head, without a weight: the two maps of head h = g * group + hg are
    rows (2 g) * group + hg and (2 g + 1) * group + hg of ``attn`` [T, 2 * n_heads * value_dim]."""
    if attn.dtype != out.dtype:
        raise KernelError("diff_combine: one element type")
    call("fx_diff_combine", _ptr(attn), _rows(attn), _ptr(out), _rows(out), code(attn), attn.shape[0], n_heads, group,
         value_dim, float(lam), float(eps), float(post), stream if stream is not None else stream_ptr())
    return out


def input_conv(x, weight, taps, tail, token_seq, seq_slot, out, update_tail=False, stream=None, add_input=True):
    """out[t] = x[t] + sum_j weight[:, j] x[t - taps + 1 + j] over the tokens of each request (``weight`` [channels,
    taps]); the inputs before the step come from ``tail`` [slots, taps - 1, channels] 32-bit.  ``update_tail``: only
    when every entry brings exactly one token; the kernel then also moves the tail on (:func:`conv_tail_update`
    otherwise).  ``add_input`` False: the sum alone."""
    if out.dtype != x.dtype or out.data_ptr() == x.data_ptr():
        raise KernelError("input_conv: an output of its own, of the input's element type")
    call("fx_input_conv", _ptr(x), code(x), _rows(x), _ptr(weight), code(weight), int(taps), _ptr(tail), _ptr(token_seq),
         _ptr(seq_slot), _ptr(out), _rows(out), x.shape[0], x.shape[1], int(update_tail), int(add_input),
         stream if stream is not None else stream_ptr())
    return out


def embed_pos(table, ids, pos_table, positions, out, status=None, stream=None):
    """out[t] = table[ids[t]] + pos_table[positions[t]] in 32 bits."""
    call("fx_embed_pos", _ptr(table), code(table), _ptr(ids), _ptr(pos_table), code(pos_table), _ptr(positions), _ptr(out),
         ids.numel(), table.shape[1], table.shape[0], pos_table.shape[0], _ptr(status),
         stream if stream is not None else stream_ptr())
    return out


def softcap_(x, cap, stream=None):
    """x = cap * tanh(x / cap) (32-bit, in place)."""
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("softcap_ takes a contiguous 32-bit tensor")
    call("fx_softcap", _ptr(x), x.numel(), float(cap), stream if stream is not None else stream_ptr())
    return x


def relu_square_(x, stream=None):
    """x = max(x, 0)^2 over rows, in place."""
    call("fx_relu_square", _ptr(x), code(x), _rows(x), x.shape[0], x.shape[1], stream if stream is not None else stream_ptr())
    return x


def rope_table(positions, inv_freq, out, stream=None, magnitude=1.0):
    """out[t, i] = magnitude * (cos, sin)(positions[t] * inv_freq[i]); out is float32 [T, half, 2]."""
    call("fx_rope_table", _ptr(positions), _ptr(inv_freq), positions.numel(), inv_freq.numel(), _ptr(out),
         float(magnitude), stream if stream is not None else stream_ptr())
    return out


def _route_extra(extra):
    """(choice bias pointer, weight scale, renorm eps) of the routing entry points; ``extra`` None: none of them."""
    bias, scale, eps = extra if extra is not None else (None, 1.0, 0.0)
    if bias is not None and (bias.dtype != torch.float32 or not bias.is_contiguous()):
        raise KernelError("routing: the choice bias is a contiguous 32-bit vector, one number per expert")
    return _ptr(bias), float(scale), float(eps)


def route_small(logits, top_k, renorm, ids, weights, offsets, src_token, inv_perm, active=None, n_experts=None,
                stream=None, extra=None):
    """router_topk and moe_align of a small step (at most 1024 tokens) in one launch.  ``extra`` = (choice_bias,
    weight_scale, renorm_eps): a 32-bit number per expert added to sigmoid(logit) for the choice only, a factor on
    the final weights, a number added to the sum the kept scores are divided by (all four routing calls take it)."""
    T, E = logits.shape[0], (n_experts or logits.shape[1])
    call("fx_route_small", _ptr(logits), _rows(logits), T, E, top_k, int(renorm), _ptr(ids), _ptr(weights), _ptr(offsets),
         _ptr(src_token), _ptr(inv_perm), _ptr(active), active.numel() if active is not None else 0,
         *_route_extra(extra), stream if stream is not None else stream_ptr())


ROUTE_FUSED_MAX_TOKENS = 8     # the kernel keeps a sum per token in registers
ROUTE_FUSED_MAX_ROWS = 1024


def route_fused_ok(x, w_route, n_experts: int, top_k: int = 1) -> bool:
    """Whether :func:`route_fused` takes these operands."""
    T, H = x.shape
    R = w_route.shape[0]
    smem = 8 * H * 2 + (8 * R + 8 * n_experts) * 4 + (2 * n_experts + 1 + 16 * top_k) * 4
    return (T <= ROUTE_FUSED_MAX_TOKENS and top_k <= 64 and x.dtype == torch.bfloat16 and w_route.dtype == torch.bfloat16
            and w_route.dim() == 2 and R <= ROUTE_FUSED_MAX_ROWS and smem <= 200 * 1024 and H % 8 == 0
            and w_route.shape[1] == H and x.stride(0) % 8 == 0 and w_route.stride(0) % 8 == 0 and x.stride(1) == 1
            and w_route.stride(1) == 1 and x.data_ptr() % 16 == 0 and w_route.data_ptr() % 16 == 0)


def route_fused(x, w_route, logits, top_k, renorm, ids, weights, offsets, src_token, inv_perm, active=None, n_experts=None,
                xp_out=None, stream=None, extra=None):
    """What stands between the norm and the experts in a step of a few tokens, in one launch of one thread-block
    cluster (see :func:`route_fused_ok`): the router's product logits = x . w_route^T (32-bit sums; ``w_route`` may carry
    rows beyond the experts', whose logits later kernels read), :func:`route_small` on the first ``n_experts`` columns
    and, with ``xp_out`` [tokens * top_k, hidden], the rows of ``x`` copied into expert order (bit 2 of ``renorm``, value
    4: each row multiplied by its routing weight on the way)."""
    T, H = x.shape
    R = w_route.shape[0]
    E = n_experts or R
    call("fx_route_fused", _ptr(x), _rows(x), _ptr(w_route), _rows(w_route), T, R, E, H, top_k, int(renorm), _ptr(logits),
         _rows(logits), _ptr(ids), _ptr(weights), _ptr(offsets), _ptr(src_token), _ptr(inv_perm), _ptr(active),
         active.numel() if active is not None else 0, _ptr(xp_out), _rows(xp_out) if xp_out is not None else 0,
         *_route_extra(extra), stream if stream is not None else stream_ptr())


ROUTE_SMALL_MAX_TOKENS = 48    # measured with 60 experts: the one-block kernel 4 to 8 us up to here, the two kernels 8 us
ROUTE_SMALL_MAX_EXPERTS = 256  # its shared memory: 32 warps x experts x 4 bytes


def route(logits, top_k, renorm, ids, weights, scratch, offsets, src_token, inv_perm, active=None, n_experts=None,
          stream=None, extra=None):
    """router_topk and moe_align of a step of any size: the top-k kernel counts each expert's rows as it chooses,
    the placing kernel sums the counts itself.  ``scratch``: 2 * n_experts int32."""
    T, E = logits.shape[0], (n_experts or logits.shape[1])
    call("fx_route", _ptr(logits), _rows(logits), T, E, top_k, int(renorm), _ptr(ids), _ptr(weights), _ptr(scratch),
         _ptr(offsets), _ptr(src_token), _ptr(inv_perm), _ptr(active), active.numel() if active is not None else 0,
         *_route_extra(extra), stream if stream is not None else stream_ptr())


PAIR_HALVES, PAIR_ADJACENT = 0, 1
ATTENTION_MAX_KEY_DIM, ATTENTION_MAX_VALUE_DIM = 640, 512    # what the general attention kernels hold of a row


def rope_kv_write(qkv, positions, token_seq, seq_slot, inv_freq, rotary_dim, k_pages, v_pages, block_table, page_size,
                  n_heads, n_kv_heads, head_dim, write_cache=True, status=None, stream=None, cos_sin=None,
                  pairing=PAIR_HALVES):
    """Rotates the q and k heads of the fused [q|k|v] rows in place at each token's position and stores k and v in
    their cache pages.  ``inv_freq`` ([rotary_dim/2] float32, or None for no rotation) gives each pair's frequency,
    ``pairing`` which elements form pair i: PAIR_HALVES (i, i + rotary_dim/2) or PAIR_ADJACENT (2i, 2i+1);
    ``cos_sin`` ([T, rotary_dim/2, 2], optional) holds this step's cos and sin, made by :func:`rope_table`."""
    T = qkv.shape[0]
    call("fx_rope_kv_write", _ptr(qkv), code(qkv), _rows(qkv), _ptr(positions), _ptr(token_seq), _ptr(seq_slot),
         _ptr(inv_freq), _ptr(cos_sin), rotary_dim, int(pairing), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1], page_size,
         T, n_heads, n_kv_heads, head_dim, int(write_cache), _ptr(status), stream if stream is not None else stream_ptr())


def paged_attention(q, k_pages, v_pages, block_table, page_size, positions, token_seq, seq_slot, out, n_heads,
                    n_kv_heads, head_dim, window, scale, stream=None, softcap=None):
    """``q`` is a [T, >= n_heads*head_dim] view whose rows start with the query heads.  ``softcap`` c: scaled
    scores pass through c * tanh(s / c) before the softmax."""
    T = q.shape[0]
    call("fx_paged_attention", _ptr(q), _rows(q), _ptr(k_pages), _ptr(v_pages), code(q), _ptr(block_table),
         block_table.shape[1], page_size, _ptr(positions), _ptr(token_seq), _ptr(seq_slot), _ptr(out), _rows(out), T,
         n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), float(softcap or 0.0),
         stream if stream is not None else stream_ptr())
    return out


def paged_attention_ex(q, ldq, ldqh, k_pages, v_pages, ldk, ldv, block_table, page_size, positions, token_seq, seq_slot,
                       out, ldo, ldoh, n_heads, n_kv_heads, key_dim, value_dim, window, scale, softcap=None, slopes=None,
                       stream=None, keep_first=0, sinks=None, value_share=1):
    """:func:`paged_attention` in its general form: keys of ``key_dim`` and values of ``value_dim`` elements whose
    positions lie ``ldk`` / ``ldv`` elements apart in their pages (values that are the leading part of the cached
    key rows: the same tensor twice with ldv = ldk); ``q`` and ``out`` are any tensors addressed by a token stride
    and a head stride; ``slopes`` (float32 [n_heads], optional): slopes[h] * (i - j) is taken off the score of key j
    for the query at position i; ``keep_first`` (with a window): the request's first positions stay visible beside
    the window; ``sinks`` (float32 [n_heads], optional): exp(sinks[h]) joins the softmax's denominator once;
    ``value_share``: that many consecutive key heads read one value head (the value pages hold n_kv_heads /
    value_share heads)."""
    T = positions.numel()
    if slopes is not None and (slopes.dtype != torch.float32 or slopes.numel() != n_heads):
        raise KernelError("paged_attention_ex: one 32-bit slope per head")
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != n_heads):
        raise KernelError("paged_attention_ex: one 32-bit sink per head")
    call("fx_paged_attention_ex", _ptr(q), int(ldq), int(ldqh), _ptr(k_pages), _ptr(v_pages), int(ldk), int(ldv), code(q),
         _ptr(block_table), block_table.shape[1], page_size, _ptr(positions), _ptr(token_seq), _ptr(seq_slot), _ptr(out),
         int(ldo), int(ldoh), T, n_heads, n_kv_heads, key_dim, value_dim, int(window or 0), float(scale),
         float(softcap or 0.0), _ptr(slopes), int(keep_first or 0), _ptr(sinks), int(value_share),
         stream if stream is not None else stream_ptr())
    return out


GENERAL_TILE_ROWS = 64     # (token, head) pairs a tile of the tensor-core kernel of the general form holds


def general_attention_ok(q, ldq, ldqh, k_pages, v_pages, ldk, ldv, out, ldo, ldoh, key_dim, value_dim,
                         kv_strides=None) -> int:
    """Whether :func:`general_attention` takes these operands (bfloat16, widths in steps of 16, 16-byte rows): 0, or
    how many of its blocks an SM holds."""
    alias = int(v_pages.data_ptr() == k_pages.data_ptr() and ldv == ldk and value_dim <= key_dim
                and (kv_strides is None or tuple(kv_strides[:2]) == tuple(kv_strides[2:])))
    if kv_strides is not None and any(int(x) % 8 for x in kv_strides):
        return 0
    return int(q.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and ldq % 8 == 0 and ldqh % 8 == 0 and ldk % 8 == 0 and ldv % 8 == 0 and ldo % 2 == 0 and ldoh % 2 == 0
            and q.data_ptr() % 16 == 0 and k_pages.data_ptr() % 16 == 0 and v_pages.data_ptr() % 16 == 0
            and out.data_ptr() % 4 == 0 and _get("fx_general_attention_ok")(key_dim, value_dim, alias))


def general_attention_fits(key_dim: int, value_dim: int) -> bool:
    """Whether the tensor-core kernel of the general form holds rows of these widths at all (separate keys and values)."""
    return bool(_get("fx_general_attention_ok")(int(key_dim), int(value_dim), 0))


def general_attention_items(entries, n_heads: int, n_kv_heads: int):
    """The work list of :func:`general_attention` for a step: int32 [n, 5] rows of (first flat token, tokens, entry,
    first query head, heads).  ``entries``: the number of tokens of each entry, in the order of the flattened batch.
    A tile holds up to GENERAL_TILE_ROWS (token, head) pairs: consecutive tokens of one entry times the heads (at
    most that many) that share one kv head."""
    import numpy as np

    group = n_heads // n_kv_heads
    n_h = min(group, GENERAL_TILE_ROWS)
    per = max(1, GENERAL_TILE_ROWS // n_h)
    out, flat = [], 0
    for b, n in enumerate(entries):
        for i in range(0, n, per):
            nt = min(per, n - i)
            for g in range(n_kv_heads):
                for c in range(0, group, GENERAL_TILE_ROWS):
                    out.append((flat + i, nt, b, g * group + c, min(GENERAL_TILE_ROWS, group - c)))
        flat += n
    out.reverse()      # the late tokens of a request see the most keys: their tiles start first
    return np.asarray(out, dtype=np.int32).reshape(-1, 5)


def general_attention(q, ldq, ldqh, k_pages, v_pages, ldk, ldv, block_table, page_size, positions, token_seq, seq_slot,
                      items, out, ldo, ldoh, n_heads, n_kv_heads, key_dim, value_dim, window, scale, slopes=None,
                      stream=None, n_splits=1, part_o=None, part_ml=None, kv_strides=None, keep_first=0, softcap=None,
                      sinks=None, value_share=1):
    """:func:`paged_attention_ex` in bfloat16 on the tensor cores (see :func:`general_attention_ok`).  ``items``: the
    device copy of :func:`general_attention_items`, or None when every entry brings one token (a tile a token and
    kv head; nothing comes from the host, so a captured step replays unchanged).  ``n_splits`` > 1 (without items):
    every token's visible keys are cut into that many runs, a block each; ``part_o`` float32 [T, heads, n_splits,
    value_dim] and ``part_ml`` float32 [T, heads, n_splits, 2] are scratch, and a second kernel adds the runs up.
    ``kv_strides`` = (k page stride, k head stride, v page stride, v head stride) in elements, for keys and values that
    do not lie [page][kv head][position][ld] (rows that hold all heads side by side); ``ldk`` / ``ldv`` stay the
    distance between two positions.  ``softcap``, ``sinks``, ``value_share``: as :func:`paged_attention_ex`."""
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != n_heads):
        raise KernelError("general_attention: one 32-bit sink per head")
    strides = (ctypes.c_long * 4)(*[int(x) for x in kv_strides]) if kv_strides is not None else None
    global _launches
    n = items.shape[0] if items is not None else positions.numel()
    if n_splits > 1:
        _launches += 1
    call("fx_general_attention", _ptr(q), int(ldq), int(ldqh), _ptr(k_pages), _ptr(v_pages), int(ldk), int(ldv),
         ctypes.cast(strides, c_void_p) if strides is not None else None, _ptr(block_table), block_table.shape[1], page_size, _ptr(positions), _ptr(token_seq), _ptr(seq_slot),
         _ptr(items), n, _ptr(out), int(ldo), int(ldoh), n_heads, n_kv_heads, key_dim, value_dim, int(window or 0),
         float(scale), _ptr(slopes), int(n_splits), _ptr(part_o), _ptr(part_ml), int(keep_first or 0),
         float(softcap or 0.0), _ptr(sinks), int(value_share), stream if stream is not None else stream_ptr())
    return out


def qk_norm_store(qkv, positions, token_seq, seq_slot, q_weight, k_weight, eps, temperature, k_pages, v_pages, block_table,
                  page_size, n_heads, n_kv_heads, key_dim, value_dim, write_cache=True, status=None, stream=None,
                  value_norm_eps=None):
    """Rows of [q heads | k heads | v heads] (widths key_dim, key_dim, value_dim), in place: q and k normed per head
    (x / sqrt(mean(x^2) + eps) * weight; weights [key_dim] or None), q times the query temperature
    1 + coef * ln(floor((pos + 1) / every) + 1) (``temperature`` = (coef, every) or None); k and v stored in their
    pages ([pages, kv heads, page, key_dim] and [.., value_dim]).  ``value_norm_eps``: every value head is divided
    by its root mean square, v / sqrt(mean(v^2) + eps), on its way into the pages."""
    coef, every = temperature if temperature is not None else (0.0, 0)
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qk_norm_store: both norm weights or none")
    call("fx_qk_norm_store", _ptr(qkv), code(qkv), _rows(qkv), _ptr(positions), _ptr(token_seq), _ptr(seq_slot),
         _ptr(q_weight), _ptr(k_weight), code(q_weight) if q_weight is not None else 0, float(eps), float(coef), int(every),
         _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1], page_size, qkv.shape[0], n_heads,
         n_kv_heads, key_dim, value_dim, int(write_cache), _ptr(status),
         float(value_norm_eps) if value_norm_eps is not None else -1.0, stream if stream is not None else stream_ptr())


def latent_prep(q, dkv, positions, token_seq, seq_slot, c_weight, eps, cos_sin, rot_dims, q_plain, q_full, pages,
                block_table, page_size, n_heads, plain_dim, rot_dim, rank, write_cache=True, status=None, stream=None,
                pairing=PAIR_ADJACENT):
    """The step between a latent attention's projections and its attention kernel: ``dkv`` rows [rank | rot_dim] become
    the cached row (the latent normed with ``c_weight``, the key part rotated by ``cos_sin`` [T, rot_dims / 2, 2] on
    neighbouring pairs or, ``pairing`` PAIR_HALVES, on pairs (i, i + rot_dims / 2)); ``q`` rows of heads [plain_dim | rot_dim] are split into ``q_plain`` [heads, T, plain_dim]
    and the rotated part in columns rank.. of ``q_full`` [heads, T, rank + rot_dim].  ``q_plain`` None (and ``q_full``
    None): the queries stay token rows and their rotated parts are turned where they lie."""
    T = q.shape[0]
    call("fx_latent_prep", _ptr(q), _rows(q), _ptr(dkv), _rows(dkv), code(q), _ptr(positions), _ptr(token_seq),
         _ptr(seq_slot), _ptr(c_weight), code(c_weight), float(eps), _ptr(cos_sin), int(rot_dims), _ptr(q_plain),
         _ptr(q_full), _ptr(pages), _ptr(block_table), block_table.shape[1], page_size, T, n_heads, plain_dim, rot_dim,
         rank, int(write_cache), _ptr(status), int(pairing), stream if stream is not None else stream_ptr())


def rmsnorm_rows(x, weight, eps, out, stream=None):
    """out = x / sqrt(mean(x^2) + eps) * weight over the rows of any 2-D views with contiguous rows (either
    element type on either side; 32-bit arithmetic)."""
    call("fx_rmsnorm_rows", _ptr(x), code(x), _rows(x), _ptr(weight), code(weight), float(eps), _ptr(out), code(out),
         _rows(out), x.shape[0], x.shape[1], stream if stream is not None else stream_ptr())
    return out


def heads_to_tokens(x, out, gate=None, stream=None, gate_per_head=False):
    """out[t, h * V + v] = x[h, t, v] (* sigmoid(gate[t, h * V + v])): rows laid out head by head back into token
    rows.  ``x`` contiguous [heads, T, V]; ``gate`` a row view of out's width, or with ``gate_per_head`` of one
    number a head (sigmoid(gate[t, h]))."""
    H, T, V = x.shape
    if not x.is_contiguous() or (gate is not None and gate.dtype != x.dtype) or out.dtype != x.dtype:
        raise KernelError("heads_to_tokens: contiguous [heads, tokens, width] and one element type")
    call("fx_heads_to_tokens", _ptr(x), V, T * V, _ptr(gate), _rows(gate) if gate is not None else 0, _ptr(out), _rows(out),
         code(x), T, H, V, int(gate_per_head), stream if stream is not None else stream_ptr())
    return out


def gate_heads_(x, gate, n_heads, stream=None, gate_per_head=False):
    """x[t, c] *= sigmoid(gate[t, c]) over token rows of ``n_heads`` heads, in place (the same kernel as
    :func:`heads_to_tokens`, reading the rows where they lie)."""
    T, W = x.shape
    if gate.dtype != x.dtype or W % n_heads:
        raise KernelError("gate_heads_: one element type, a width that the heads divide")
    call("fx_heads_to_tokens", _ptr(x), _rows(x), W // n_heads, _ptr(gate), _rows(gate), _ptr(x), _rows(x), code(x), T,
         n_heads, W // n_heads, int(gate_per_head), stream if stream is not None else stream_ptr())
    return x


PREFILL_TILE = 64


def prefill_attention(q, k_pages, v_pages, block_table, page_size, tiles, seq_slot, out, n_heads, n_kv_heads, head_dim,
                      window, scale, stream=None, softcap=None):
    """Flash attention of prompt portions (bfloat16).  ``tiles``: int32 [n, 4] rows of
    (first flat token, rows <= 64, entry index, absolute position of the first row)."""
    if q.dtype != torch.bfloat16:
        raise KernelError("prefill_attention is a bfloat16 kernel")
    call("fx_prefill_attention", _ptr(q), _rows(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
         block_table.shape[1], page_size, _ptr(tiles), tiles.shape[0], _ptr(seq_slot), _ptr(out), _rows(out), n_heads,
         n_kv_heads, head_dim, int(window or 0), float(scale), float(softcap or 0.0),
         stream if stream is not None else stream_ptr())
    return out


WIDE_PREFILL_TILE = 256


def prefill_ok(q, out, k_pages, head_dim) -> bool:
    """Whether the mma.sync prompt attention kernel takes these operands (bfloat16, head sizes in steps of 16)."""
    return (q.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and 0 < head_dim <= 256 and head_dim % 16 == 0
            and q.stride(0) % 8 == 0 and out.stride(0) % 2 == 0 and q.data_ptr() % 16 == 0 and k_pages.data_ptr() % 16 == 0)


def prefill_tc_ok(q, out, k_pages, page_size, head_dim) -> bool:
    """Whether the tcgen05 prompt attention kernel takes these operands."""
    return (q.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and head_dim in (64, 128)
            and page_size >= 64 and page_size % 64 == 0 and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


PREFILL_KEY_BLOCK = 128          # positions per key block of the tcgen05 prompt attention kernel
PREFILL_MAX_RUNS = 32            # runs of key blocks a tile may be cut into (a lane of the merging warp each)
# The planner's cost model, in units of the time a block of 128 keys takes a tile (measured on a B200, 16 heads of
# 128: 2.7 us): what an item costs beside its key blocks (set-up, the first block's latency, its output), and the
# second kernel that adds the runs of cut tiles up.
PREFILL_ITEM_OVERHEAD, PREFILL_MERGE_COST = 5, 3
PREFILL_RUN_CHOICES = (0, 16, 12, 8, 6, 4)   # key blocks a run (0: tiles stay whole)


def _prefill_items(tiles, run: int):
    items, merges, parts = [], [], 0
    for tok0, rows, b, pos0, first, end in tiles:
        n_blk = end - first
        runs = min(PREFILL_MAX_RUNS, -(-n_blk // run)) if run > 0 else 1
        if runs <= 1:
            items.append((tok0, rows, b, pos0, first, end, -1, 0))
            continue
        per = -(-n_blk // runs)
        first_part = parts
        for kb in range(first, end, per):
            items.append((tok0, rows, b, pos0, kb, min(end, kb + per), parts, 0))
            parts += 1
        merges.append((tok0, rows, first_part, parts - first_part))
    items.sort(key=lambda it: it[4] - it[5])      # most key blocks first (stable: ties stay in order)
    return items, merges, parts


def _prefill_makespan(items, parts: int, n_heads: int, sms: int) -> float:
    """How long the items take on ``sms`` SMs that take them heaviest first, each head its own copy of every item:
    no less than the heaviest item, than an even share of all work, and than the two items that must share an SM once
    there are more items than SMs; plus the adding up of the parts."""
    costs = [it[5] - it[4] + PREFILL_ITEM_OVERHEAD for it in items]           # descending already
    n = len(costs) * n_heads
    est = max(costs[0], sum(costs) * n_heads / sms)
    if n > sms:
        est = max(est, costs[(sms - 1) // n_heads] + costs[sms // n_heads])
    return est + (PREFILL_MERGE_COST if parts else 0)


def prefill_tc_plan(entries, window, n_heads: int, sms: int = 0, run_blocks: int = -1):
    """The work items of the tcgen05 prompt attention kernel for a step.  ``entries``: (tokens, first position) of
    each entry, in the order of the flattened batch.  A tile is up to 256 queries of one entry; it sees the key blocks
    (of 128 positions) from its first query's first visible key to its last query's own.  Tiles with many key blocks
    may be cut into runs whose partial results a second kernel adds up: a portion behind a long cached prefix is one
    tile with all the keys, and without the cut it would keep as many SMs busy as there are heads.  A cut item costs
    (PREFILL_ITEM_OVERHEAD), so the run length is the one of PREFILL_RUN_CHOICES whose items finish first by
    :func:`_prefill_makespan`, and whole tiles stay unless a cut is 15 % faster by that estimate.  Returns (items int32 [n, 8], merges int32 [m, 4], parts) as
    ``fx_prefill_attention_tc`` takes them: heavy items first; a tile's runs have consecutive parts in the order of
    their keys.  ``run_blocks`` >= 0: this many key blocks a run instead of the choice (0: no cut; tests)."""
    import numpy as np

    sms = sms or sm_count()
    W = int(window or 0)
    tiles, flat = [], 0
    for b, (n, start) in enumerate(entries):
        for i in range(0, n, WIDE_PREFILL_TILE):
            rows, pos0 = min(WIDE_PREFILL_TILE, n - i), start + i
            first = (max(0, pos0 - W + 1) if W > 0 else 0) // PREFILL_KEY_BLOCK
            end = (pos0 + rows - 1) // PREFILL_KEY_BLOCK + 1
            tiles.append((flat + i, rows, b, pos0, first, end))
        flat += n
    best = first = None
    whole = 0.0
    for run in (PREFILL_RUN_CHOICES if run_blocks < 0 else (run_blocks,)):
        items, merges, parts = _prefill_items(tiles, run)
        if run > 0 and not parts and best is not None:
            continue                                  # nothing was cut: the same items as the whole tiles
        est = _prefill_makespan(items, parts, n_heads, sms)
        # (whole tiles stay unless a cut promises a clear gain: the model is good to a tenth or so)
        if best is None or est < (0.85 * whole if best[1] is first else best[0] - 1e-9):
            best = (est, items, merges, parts)
            if first is None:
                first, whole = items, est
    _, items, merges, parts = best
    return (np.asarray(items, dtype=np.int32).reshape(-1, 8), np.asarray(merges, dtype=np.int32).reshape(-1, 4), parts)


def prefill_attention_tc(q, k_pages, v_pages, block_table, page_size, items, seq_slot, out, n_heads, n_kv_heads,
                         head_dim, window, scale, status=None, stream=None, merges=None, part_o=None, part_ml=None):
    """Flash attention of prompt portions on the tcgen05 tensor cores (bfloat16, head_dim 64 or 128, pages of a
    multiple of 64 positions).  ``items``, ``merges``: device copies of what :func:`prefill_tc_plan` returns;
    ``part_o`` float32 [parts, n_heads, 256, head_dim] and ``part_ml`` float32 [parts, n_heads, 256, 2]: scratch for the
    tiles that were cut into runs of key blocks (a second kernel adds the runs up)."""
    global _launches
    n_merges = merges.shape[0] if merges is not None else 0
    if n_merges:
        _launches += 1
    call("fx_prefill_attention_tc", _ptr(q), _rows(q), q.shape[0], _ptr(k_pages), _ptr(v_pages), k_pages.shape[0],
         _ptr(block_table), block_table.shape[1], page_size, _ptr(items), items.shape[0], _ptr(seq_slot), _ptr(out),
         _rows(out), n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), _ptr(status),
         _ptr(part_o) if n_merges else None, _ptr(part_ml) if n_merges else None, _ptr(merges) if n_merges else None,
         n_merges, stream if stream is not None else stream_ptr())
    return out


def router_topk(logits, top_k, renorm, ids, weights, n_experts=None, stream=None, extra=None):
    """``n_experts``: the first columns of ``logits`` that are router logits (default: all).  ``extra``: see
    :func:`route_small`."""
    T, E = logits.shape[0], (n_experts or logits.shape[1])
    call("fx_router_topk", _ptr(logits), _rows(logits), T, E, top_k, int(renorm), _ptr(ids), _ptr(weights),
         *_route_extra(extra), stream if stream is not None else stream_ptr())


def moe_align(ids, n_experts, scratch, offsets, src_token, inv_perm, active=None, stream=None):
    """``active`` (optional, int32 [n_slots]) receives the experts that got rows, then -1."""
    T, K = ids.shape
    call("fx_moe_align", _ptr(ids), T, K, n_experts, _ptr(scratch), _ptr(offsets), _ptr(src_token), _ptr(inv_perm),
         _ptr(active), active.numel() if active is not None else 0, stream if stream is not None else stream_ptr())


SKINNY_MAX_TOKENS = 64


def skinny_ok(x, w) -> bool:
    """Whether the decode-sized product kernel takes these operands."""
    K = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 32 == 0 and x.stride(0) % 8 == 0
            and w.stride(-2) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(x, w, out, *, bias=None, accumulate=False, gated=False, unary=None, x_rows=None, group_offsets=None,
                active_groups=None, tokens_hint=0, transposed_out=False, stream=None):
    """out[rows, N] (+)= x . w^T for few rows: streams ``w`` once.  ``gated``: ``w`` is
    [gate rows ; up rows] (2N rows) and out = silu(gate) * up.  Grouped: ``w`` is
    [G, rows, K], ``group_offsets``/``active_groups`` come from :func:`moe_align`."""
    rows, N = (out.shape[1], out.shape[0]) if transposed_out else out.shape   # transposed: out is [N, rows]
    K = x.shape[1]
    if group_offsets is not None:
        wrows, wstride, ldw = w.shape[1], w.stride(0), w.stride(1)
        n_slots = active_groups.numel()
    else:
        wrows, wstride, ldw = w.shape[0], 0, w.stride(0)
        n_slots = 1
    gated, lim, alpha = _gate_args(gated)
    if wrows != (2 * N if gated else N) or w.shape[-1] != K:
        raise KernelError(f"gemm_skinny shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call("fx_gemm_skinny", _ptr(x), _rows(x), _ptr(x_rows), _ptr(w), ldw, wstride, _ptr(bias),
         code(bias) if bias is not None else 0, _ptr(out), code(out), _rows(out), int(accumulate), rows, N, K,
         int(_gated_or_unary(gated, unary)), N if gated else 0, lim, alpha, _ptr(group_offsets), _ptr(active_groups), n_slots, int(tokens_hint),
         int(transposed_out), stream if stream is not None else stream_ptr())
    return out


SLAB_MAX_TOKENS = 32      # the kernel walks its tokens 8 at a time over a matrix it holds in shared memory
# up to here it is the faster one (measured on a B200, 8 layers' decode step: 16 tokens 1,728 against 1,742 us, 24 tokens
# 2,271 against 2,221, 32 tokens 2,449 against 2,353; 1 to 8 tokens 1 to 2 % faster)
SLAB_BETTER_MAX_TOKENS = 16


def slab_ok(x, w) -> bool:
    """Whether :func:`gemm_slab` takes the product: bfloat16, few tokens, a plain matrix that fits the shared
    memory of all SMs together (a slab of rows a block), K a multiple of 128, rows 16-byte aligned."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.dim() != 2 or x.shape[0] > SLAB_MAX_TOKENS:
        return False
    if x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or x.stride(1) != 1 or w.stride(1) != 1:
        return False
    return bool(_get("fx_gemm_slab_ok")(w.shape[0], w.shape[1], x.shape[0]))


def gemm_slab(x, w, out, *, bias=None, accumulate=False, status=None, stream=None):
    """out[T, N] (+)= x . w^T (+ bias) by the kernel that asks for its whole slab of ``w`` before it waits for the
    kernel before it on the stream (gemm_slab.cu): for a matrix that kernel did not write."""
    T, K = x.shape
    N = w.shape[0]
    if out.shape != (T, N) or w.shape[1] != K:
        raise KernelError(f"gemm_slab shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call("fx_gemm_slab", _ptr(x), _rows(x), _ptr(w), w.stride(0), _ptr(bias), code(bias) if bias is not None else 0,
         _ptr(out), code(out), _rows(out), int(accumulate), T, N, K, _ptr(status),
         stream if stream is not None else stream_ptr())
    return out


DECODE_BLOCK_OVERHEAD = 128       # start and end of a block, in keys' worth of a block's time
DECODE_MERGE_COST = 256           # the merge of the key ranges, in the same unit
DECODE_BLOCKS_TO_SATURATE = 160   # blocks streaming at the same time that draw the machine's whole bandwidth
DECODE_MAX_SPLITS = 16
DECODE_RUN_LATENCY = 0.15         # share of a run's length that a block's own chain of tiles adds


def decode_tma_blocks_per_sm(dtype, head_dim: int, page_size: int) -> int:
    """Blocks an SM holds of the decode attention kernel that streams pages by TMA (attention_decode_tma.cu);
    0 where it does not apply (then the cp.async kernel runs, three blocks an SM).  Mirrors the kernel's ring:
    stages of 2 x head_dim x 64 x 2 bytes, as many as fit 96 KB (at least 3, at most 8)."""
    if dtype != torch.bfloat16 or head_dim <= 0 or head_dim % 64 or head_dim > 256 or page_size < 64 or page_size % 64:
        return 0
    stage = 2 * (head_dim // 64) * 8192
    stages = max(3, min(8, (96 * 1024) // stage))
    smem = 1024 + max(stages * stage, 4 * 16 * (head_dim + 8) * 4) + 16 * (head_dim * 2 + 16)
    return min(2, (227 * 1024) // (smem + 1024))


def decode_split_plan(n_tokens: int, n_kv_blocks: int, max_positions: int, blocks_per_sm: int = 3,
                      single_is_final: bool = False, run_latency: float = 0.0):
    """(split_len, n_splits) for :func:`decode_attention`.  split_len 0: every token's visible keys are cut
    into n_splits runs of equal length, so that all blocks have work whatever the context length is.
    n_splits is a function of the step's size and the context limit only (a CUDA graph keeps its grid).  The cost
    of n runs, in the time one block takes for a key: the keys stream at the rate of the whole machine
    (DECODE_BLOCKS_TO_SATURATE blocks' worth) or, with few or unevenly many blocks, at the rate of the blocks of a
    wave one after the other; every wave pays a block's start and end and a share of a run's length (a block's own
    chain of tiles, which nothing hides at its start and its end); more than one run pays the merge
    (``single_is_final``: a kernel that writes a single run's result itself, so only n > 1 pays it).
    ``run_latency``: the share of a run's length counted once more per wave; the kernel that streams pages by TMA is
    planned with DECODE_RUN_LATENCY.  Measured with it on a B200 with 16 kv heads of 128, context 2,048 of 4,096, 8
    layers' step in microseconds: 3 requests 864 with 4 runs and 848 with 6; 4 requests 956 with 3 and 936 with 4;
    5 requests 1,081 with 2 and 1,046 with 3; 6 requests 1,167 with 2 and 1,133 with 3; 8 requests 1,258 with 2 and
    1,357 with 3 (384 blocks where 296 fit); 9 requests 1,482 with 1, 1,376 with 2, 1,464 with 3."""
    blocks = max(1, n_tokens * n_kv_blocks)
    slots = sm_count() * blocks_per_sm
    best, best_cost = 1, None
    for n in range(1, min(DECODE_MAX_SPLITS, max(1, -(-max_positions // 64))) + 1):
        waves = -(-blocks * n // slots)
        stream = max(blocks * max_positions / DECODE_BLOCKS_TO_SATURATE, waves * max_positions / n)
        cost = (stream + waves * (DECODE_BLOCK_OVERHEAD + run_latency * max_positions / n)
                + (DECODE_MERGE_COST if n > 1 or not single_is_final else 0))
        if best_cost is None or cost < best_cost * 0.98:   # more runs only for a clear gain
            best, best_cost = n, cost
    return 0, best


def decode_store_ok(qkv, k_pages, head_dim: int, page_size: int) -> bool:
    """Whether :func:`decode_attention` can rotate and store the step's own keys and values itself (``store_new``):
    where the kernel that streams pages by TMA runs."""
    return (decode_tma_blocks_per_sm(qkv.dtype, head_dim, page_size) > 0 and k_pages.dtype == torch.bfloat16
            and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0 and k_pages.data_ptr() % 16 == 0)


def decode_attention(q, k_pages, v_pages, block_table, page_size, positions, token_seq, seq_slot, out, n_heads,
                     n_kv_heads, head_dim, window, scale, split_len, n_splits, part_acc, part_ml, status=None,
                     counters=None, stream=None, fresh_positions=0, store_new=False, write_pages=True, cos_sin=None,
                     softcap=None):
    """``softcap`` c: the scaled scores pass through c * tanh(s / c) (the kernel that streams pages by TMA does not
    take one: the call goes to the others).  ``counters``: zeroed int32 scratch that the call leaves zeroed, at least tokens x ceil(group / 16) x kv heads;
    with it the kernel that streams pages by TMA merges the key ranges itself (one kernel instead of two).
    ``fresh_positions``: 0 assumes nothing about the kernel launched just before on the stream.  N > 0 promises that
    that kernel wrote, of all this call reads, only the queries and the keys and values of at most the last N
    positions of each request; older keys are then fetched while it still runs (a false promise reads stale keys).
    ``store_new`` (one token a request; see :func:`decode_store_ok`): ``q`` is the fused [q | k | v] rows as the
    projection left them and the kernel does the rotary kernel's work itself: queries and each token's own key
    rotated (split-half pairs over the whole head, ``cos_sin`` from :func:`rope_table`; None: no rotation), key and
    value put where the attention reads them and, if ``write_pages``, into the pages."""
    global _launches
    T = q.shape[0]
    per_sm = 0 if softcap else decode_tma_blocks_per_sm(q.dtype, head_dim, page_size)
    blocks = T * n_kv_heads * -(-(n_heads // n_kv_heads) // 16)
    # Merging in the kernel pays while all blocks run at the same time: the count and the fence lengthen the end of
    # every block, which costs nothing only where no other block waits for its place.
    if counters is not None and not (per_sm > 0 and 1 < n_splits <= 32 and counters.numel() >= blocks
                                     and blocks * n_splits <= sm_count() * per_sm):
        counters = None
    if per_sm > 0 and (counters is not None or n_splits == 1):
        _launches -= 1      # no merge kernel
    call("fx_decode_attention", _ptr(q), _rows(q), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], code(q),
         _ptr(block_table), block_table.shape[1], page_size, _ptr(positions), _ptr(token_seq), _ptr(seq_slot),
         _ptr(out), _rows(out), _ptr(part_acc), _ptr(part_ml), T, n_heads, n_kv_heads, head_dim, int(window or 0),
         float(scale), split_len, n_splits, _ptr(status), _ptr(counters), int(fresh_positions), int(store_new),
         int(write_pages), _ptr(cos_sin), float(softcap or 0.0), stream if stream is not None else stream_ptr())
    return out


def decode_ok(q, head_dim: int) -> bool:
    """Whether the split-key kernels take these operands (heads of whole 16-byte vectors, aligned rows)."""
    n = 8 if q.dtype == torch.bfloat16 else 4
    return head_dim % n == 0 and q.stride(0) % n == 0 and q.data_ptr() % 16 == 0


TC_MAX_GROUPS = 1024        # experts the grouped tcgen05 kernel keeps its tile table for (gemm_tc.cu)
TC_SWAP_MAX_GROUPS = 512    # and the swapped-role kernel (gemm_tc_swap.cu)


def tc_ok(x, w) -> bool:
    """Whether the tcgen05 kernel takes these operands (bfloat16, 16-byte aligned rows)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and w.stride(-2) % 8 == 0 and (w.dim() == 2 or w.stride(0) % 8 == 0) and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and x.stride(1) == 1 and w.stride(-1) == 1)


def gemm_tc(x, w, out, *, bias=None, accumulate=False, gated=False, unary=None, group_offsets=None, status=None, stream=None):
    """out[M, N] (+)= x . w^T on the tcgen05 tensor cores.  ``gated``: ``w`` is [gate rows ; up rows] and
    out = silu(gate) * up.  Grouped: ``w`` is [G, rows, K] and the rows of ``x``/``out`` are sorted by group."""
    M, N = out.shape
    K = x.shape[1]
    if group_offsets is not None:
        G, wrows, ldw, wstride = w.shape[0], w.shape[1], w.stride(1), w.stride(0)
    else:
        G, wrows, ldw, wstride = 0, w.shape[0], w.stride(0), 0
    gated, lim, alpha = _gate_args(gated)
    if wrows != (2 * N if gated else N) or w.shape[-1] != K or x.shape[0] != M:
        raise KernelError(f"gemm_tc shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call("fx_gemm_tc", _ptr(x), _rows(x), _ptr(w), ldw, wstride, wrows, _ptr(bias), code(bias) if bias is not None else 0,
         _ptr(out), code(out), _rows(out), int(accumulate), M, N, K, int(_gated_or_unary(gated, unary)), N if gated else 0, lim, alpha,
         _ptr(group_offsets), G, _ptr(status), stream if stream is not None else stream_ptr())
    return out


def gemm_tc_swap(x, w, out, *, bias=None, accumulate=False, gated=False, unary=None, group_offsets=None, tokens_per_tile=0,
                 weights_first=None, k_splits=1, status=None, stream=None):
    """The same product as :func:`gemm_tc` with the roles swapped: 128 features of ``w`` fill the lanes of a tile,
    the tokens its columns (multiples of 16 up to ``tokens_per_tile``: 32, 64 or 128; 0 = chosen from the sizes).
    For few tokens per weight matrix: decode batches beyond the weight-streaming kernel's, experts of a prompt.
    ``weights_first``: the kernel may fetch its first weights before the kernel launched just before it has finished;
    true by default for dense products, and for grouped ones only if the caller says that ``group_offsets`` is older
    than that kernel.  ``k_splits`` > 1 (plain dense products): K is cut into runs taken by separate CTAs and a second
    kernel adds the partial sums in run order, for matrices of too few rows to fill the machine with tiles."""
    M, N = out.shape
    K = x.shape[1]
    if group_offsets is not None:
        G, wrows, ldw, wstride = w.shape[0], w.shape[1], w.stride(1), w.stride(0)
    else:
        G, wrows, ldw, wstride = 0, w.shape[0], w.stride(0), 0
    gated, lim, alpha = _gate_args(gated)
    if wrows != (2 * N if gated else N) or w.shape[-1] != K or x.shape[0] != M:
        raise KernelError(f"gemm_tc_swap shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call("fx_gemm_tc_swap", _ptr(x), _rows(x), _ptr(w), ldw, wstride, wrows, _ptr(bias), code(bias) if bias is not None else 0,
         _ptr(out), code(out), _rows(out), int(accumulate), M, N, K, int(_gated_or_unary(gated, unary)), N if gated else 0, lim, alpha,
         _ptr(group_offsets), G, int(tokens_per_tile),
         int(group_offsets is None if weights_first is None else weights_first), int(k_splits),
         _ptr(torch.empty(k_splits, M, N, dtype=torch.float32, device=out.device)) if k_splits > 1 else None,
         _ptr(status), stream if stream is not None else stream_ptr())
    return out


def gemm_tc2(x, w, out, *, bias=None, accumulate=False, gated=False, unary=None, status=None, stream=None):
    """The dense product of :func:`gemm_tc` on pairs of SMs (tcgen05 cta_group::2: 256 x 256 tiles shared by the two
    CTAs of a cluster, each fetching half of the tile's operands).  For prompt-sized dense products."""
    M, N = out.shape
    K = x.shape[1]
    gated, lim, alpha = _gate_args(gated)
    if w.dim() != 2 or w.shape[0] != (2 * N if gated else N) or w.shape[1] != K or x.shape[0] != M:
        raise KernelError(f"gemm_tc2 shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call("fx_gemm_tc2", _ptr(x), _rows(x), _ptr(w), w.stride(0), w.shape[0], _ptr(bias), code(bias) if bias is not None else 0,
         _ptr(out), code(out), _rows(out), int(accumulate), M, N, K, int(_gated_or_unary(gated, unary)), N if gated else 0, lim, alpha,
         _ptr(status), stream if stream is not None else stream_ptr())
    return out


def gather_rows(x, rows, out, stream=None):
    call("fx_gather_rows", _ptr(x), _rows(x), _ptr(rows), _ptr(out), _rows(out), code(x), out.shape[0], x.shape[1],
         stream if stream is not None else stream_ptr())
    return out


def gather_rows_scaled(x, rows, inv_perm, weights, out, stream=None):
    """out[r] = w * x[rows[r]], w the routing weight of the (token, rank) pair whose row in expert order is r
    (``inv_perm`` [T, top_k] gives each pair's row, ``weights`` [T, top_k] its weight)."""
    call("fx_gather_rows_scaled", _ptr(x), _rows(x), _ptr(rows), _ptr(inv_perm), _ptr(weights), weights.shape[1],
         _ptr(out), _rows(out), code(x), out.shape[0], x.shape[1], stream if stream is not None else stream_ptr())
    return out


def swap_better(T: int, N: int, K: int) -> bool:
    """Few tokens against a weight matrix: whether the tcgen05 kernel with the roles swapped (features in the
    lanes, tokens in the columns, weights by TMA) beats the weight-streaming mma.sync kernel.  Measured on a
    B200: beyond 32 tokens for matrices of a few thousand rows, from 8 tokens on for very large ones (the
    vocabulary head); matrices of few rows give the swapped kernel too few tiles."""
    return (T > 32 and N >= 4096) or (T >= 8 and N * K >= (1 << 27))


def pairs_better(M: int, N: int, gated: bool = False) -> bool:
    """Prompt-sized dense products: whether the kernel on pairs of SMs (256 x 256 tiles) beats the one with a CTA per
    128 x 256 tile.  Measured on a B200: from two rounds of tiles for the 74 pairs on (3 to 13 % faster, more with more
    rows); with fewer tiles than SMs the pairs leave SMs idle."""
    tiles = -(-M // 256) * -(-N // (128 if gated else 256))
    return M >= 1024 and tiles >= sm_count()


def swap_k_splits(T: int, N: int, K: int) -> int:
    """Runs of K for the swapped-role kernel on a plain dense product of few tokens, or 0 where the weight-streaming
    kernel is as good.  A matrix of N rows gives N / 128 tiles; with fewer than the machine has SMs, K is cut so that
    some 150 to 300 CTAs stream it.  Measured on a B200 (decode batches of 32 and 64): ahead from 33 tokens on, and from
    17 tokens for matrices of 8M elements and more."""
    if T > 32 or (T > 16 and N * K >= (1 << 23)):
        tiles = -(-N // 128) * -(-T // (32 if T <= 32 else 64))
        return max(1, min(8, K // 256, round(192 / tiles)))
    return 0


def _apply_unary_(out, activation, stream=None):
    """The activation of :func:`linear` as a step of its own, for the kernels that do not have it in their epilogue."""
    unary_code(activation)
    return relu_square_(out, stream=stream)


def linear(x, w, out, *, bias=None, accumulate=False, status=None, stream=None, after_short_kernel=False, activation=None):
    """out (+)= act(x . w^T (+ bias)): picks the kernel by size and element type.  ``after_short_kernel``: the kernel
    before this one on the stream is short and leaves the memory system idle; a few tokens then go to the kernel that
    asks for the whole matrix before it waits for that kernel (:func:`gemm_slab`), where the matrix fits.
    ``activation`` (None or "relu_square", not with ``accumulate``): in the product's epilogue where the chosen kernel
    has one for it, as a step of its own on ``out`` otherwise."""
    T = x.shape[0]
    act = activation
    if act is not None:
        unary_code(act)
        if accumulate:
            raise KernelError("linear: an activation on a sum that is added to what is there is not defined here")
    if after_short_kernel and T <= SLAB_BETTER_MAX_TOKENS and slab_ok(x, w) and out.dtype in _CODES:
        gemm_slab(x, w, out, bias=bias, accumulate=accumulate, status=status, stream=stream)
        return _apply_unary_(out, act, stream) if act else out
    if (T > SKINNY_MAX_TOKENS and w.shape[0] <= SKINNY_MAX_TOKENS and bias is None and skinny_ok(w, x)):
        # many tokens, a narrow output (router logits): the weight-streaming kernel with the roles swapped,
        # x streamed once as the "matrix", w as the few "tokens", stored transposed
        gemm_skinny(w, x, out, accumulate=accumulate, transposed_out=True, stream=stream)
        return _apply_unary_(out, act, stream) if act else out
    if T <= SKINNY_MAX_TOKENS and w.dim() == 2 and tc_ok(x, w):
        N, K = w.shape
        if T >= 8 and N * K >= (1 << 27):   # the vocabulary head: tiles enough without cutting K
            return gemm_tc_swap(x, w, out, bias=bias, accumulate=accumulate, unary=act, status=status, stream=stream)
        ks = swap_k_splits(T, N, K)
        if ks > 1:      # the runs' partial sums are added by a second kernel: the activation follows that
            gemm_tc_swap(x, w, out, bias=bias, accumulate=accumulate, k_splits=ks, status=status, stream=stream)
            return _apply_unary_(out, act, stream) if act else out
        if ks:
            return gemm_tc_swap(x, w, out, bias=bias, accumulate=accumulate, unary=act, status=status, stream=stream)
    if T <= SKINNY_MAX_TOKENS and skinny_ok(x, w):
        return gemm_skinny(x, w, out, bias=bias, accumulate=accumulate, unary=act, stream=stream)
    if T > SKINNY_MAX_TOKENS and tc_ok(x, w):
        if w.dim() == 2 and pairs_better(T, w.shape[0]):
            return gemm_tc2(x, w, out, bias=bias, accumulate=accumulate, unary=act, status=status, stream=stream)
        return gemm_tc(x, w, out, bias=bias, accumulate=accumulate, unary=act, status=status, stream=stream)
    gemm(x, w, out, bias=bias, accumulate=accumulate, stream=stream)
    return _apply_unary_(out, act, stream) if act else out


def gated_linear(x, w_gu, out, *, status=None, stream=None, activation="silu", bias=None):
    """out = act(x . gate^T (+ b_gate)) * (x . up^T (+ b_up)) with ``w_gu`` = [gate rows ; up rows], ``bias`` =
    [b_gate ; b_up] or None, and act SiLU or ReLU (``activation``): picks the kernel as :func:`linear` does; the
    gate|up intermediate reaches memory only on the CUDA-core path."""
    T, I = out.shape
    gated = gated_arg(activation)     # the kernels' argument: 0 plain, 1 SiLU gate, 2 ReLU gate, (3, limit, alpha)
    if bias is not None and bias.numel() != 2 * I:
        raise KernelError("gated_linear: the bias holds the gate rows' values, then the up rows'")
    if T <= SKINNY_MAX_TOKENS and tc_ok(x, w_gu) and swap_better(T, 2 * I, x.shape[1]):
        return gemm_tc_swap(x, w_gu, out, bias=bias, gated=gated, status=status, stream=stream)
    if T <= SKINNY_MAX_TOKENS and skinny_ok(x, w_gu):
        return gemm_skinny(x, w_gu, out, bias=bias, gated=gated, stream=stream)
    if T > SKINNY_MAX_TOKENS and tc_ok(x, w_gu):
        if w_gu.dim() == 2 and pairs_better(T, I, gated=True):
            return gemm_tc2(x, w_gu, out, bias=bias, gated=gated, status=status, stream=stream)
        return gemm_tc(x, w_gu, out, bias=bias, gated=gated, status=status, stream=stream)
    gu = torch.empty(T, 2 * I, dtype=out.dtype, device=out.device)
    gemm(x, w_gu, gu, bias=bias, stream=stream)
    return silu_mul(gu, out, stream=stream, activation=activation)


def combine_norm_ok(h, y) -> bool:
    """Whether :func:`moe_combine` can also write the normed rows (a thread keeps its part of a row in registers)."""
    vw = 4 if y.dtype == torch.float32 else 8
    H = h.shape[1]
    return y.dtype in _CODES and H % vw == 0 and H // vw <= 4 * 256


def moe_combine(h, y, inv_perm, topk_w, shared=None, shared_gate_logit=None, stream=None, norm=None, top_k=None):
    """h[t] += sum_k topk_w[t, k] * y[inv_perm[t, k]] (+ sigmoid(gate logit) * shared[t]).  ``norm`` = (weight, eps,
    out): also out[t] = rmsnorm(h[t]) * weight on the new rows, in the same kernel (see :func:`combine_norm_ok`).
    ``topk_w`` None (then ``top_k`` says how many rows a token has): the rows are added as they are, for experts
    whose routing weight went into their input."""
    T, H = h.shape
    top_k = topk_w.shape[1] if topk_w is not None else int(top_k)
    if norm is not None:
        w, eps, out = norm
        call("fx_moe_combine_norm", _ptr(h), _ptr(y), code(y), _ptr(inv_perm), _ptr(topk_w), top_k,
             _ptr(shared), _ptr(shared_gate_logit), shared_gate_logit.stride(0) if shared_gate_logit is not None else 0,
             T, H, _ptr(w), code(w), float(eps), _ptr(out), stream if stream is not None else stream_ptr())
        return out
    call("fx_moe_combine", _ptr(h), _ptr(y), code(y), _ptr(inv_perm), _ptr(topk_w), top_k, _ptr(shared),
         _ptr(shared_gate_logit), shared_gate_logit.stride(0) if shared_gate_logit is not None else 0, T, H, stream if stream is not None else stream_ptr())


def residual_add(h, y, stream=None):
    call("fx_residual_add", _ptr(h), _ptr(y), code(y), h.numel(), stream if stream is not None else stream_ptr())


def argmax(logits, out, stream=None):
    n, V = logits.shape
    call("fx_argmax", _ptr(logits), _rows(logits), n, V, _ptr(out), stream if stream is not None else stream_ptr())
    return out


def repetition_penalty(work, history, hist_offsets, penalty, stream=None):
    n, V = work.shape
    call("fx_repetition_penalty", _ptr(work), _rows(work), n, V, _ptr(history), _ptr(hist_offsets), _ptr(penalty),
         stream if stream is not None else stream_ptr())


def sample_or(scores, work, temperature, top_k, top_p, draw, use_sample, instead, out, stream=None):
    """Row r of ``out``: a sample of ``scores[r]`` as :func:`sample` draws it if ``use_sample[r]``, else ``instead[r]``
    (also when every candidate was filtered away).  ``scores`` stay untouched; ``work`` is scratch of the same shape."""
    n, V = scores.shape
    call("fx_sample_or", _ptr(scores), _rows(scores), _ptr(work), _rows(work), n, V, _ptr(temperature), _ptr(top_k),
         _ptr(top_p), _ptr(draw), _ptr(use_sample), _ptr(instead), _ptr(out),
         stream if stream is not None else stream_ptr())
    return out


def random_normal(out, key: int, mean: float, std: float, stream=None):
    """out[i] = mean + std * z_i, z the standard normal stream of the 64-bit ``key`` (the rule of
    ``weights.random_init``, which states it for the CPU bit for bit).  ``out``: contiguous float32 or bfloat16."""
    if not out.is_contiguous():
        raise KernelError("random_normal fills contiguous tensors")
    call("fx_random_normal", _ptr(out), code(out), out.numel(), key & ((1 << 64) - 1), float(mean), float(std),
         stream if stream is not None else stream_ptr())
    return out


def sample(work, temperature, top_k, top_p, draw, out, stream=None):
    n, V = work.shape
    call("fx_sample", _ptr(work), _rows(work), n, V, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(draw), _ptr(out),
         stream if stream is not None else stream_ptr())
    return out


def grouped_linear(x, w, out, offsets, active, rows_per_group: int, *, status=None, stream=None):
    """out[r] = x[r] . w[g]^T for the rows r of group g (``offsets`` int32 [G + 1] on the device, rows sorted by
    group; ``w`` [G, N, K]; ``out`` may have a wider row stride than N).  ``active`` lists the groups that have rows
    (int32, then -1), ``rows_per_group`` is the mean number of rows a group has, by which the kernel is chosen as the
    experts' products choose theirs."""
    T = x.shape[0]
    G, N, K = w.shape
    if tc_ok(x, w) and K % 8 == 0 and N % 8 == 0 and G <= TC_MAX_GROUPS and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0:
        if rows_per_group > 16 or G > TC_SWAP_MAX_GROUPS:
            return gemm_tc(x, w, out, group_offsets=offsets, status=status, stream=stream)
        if rows_per_group >= 8 or not (skinny_ok(x, w) and active is not None):
            return gemm_tc_swap(x, w, out, group_offsets=offsets, tokens_per_tile=32 if rows_per_group <= 8 else 64,
                                weights_first=True, status=status, stream=stream)
    if rows_per_group <= SKINNY_MAX_TOKENS and skinny_ok(x, w) and active is not None:
        return gemm_skinny(x, w, out, group_offsets=offsets, active_groups=active, tokens_hint=rows_per_group, stream=stream)
    return gemm(x, w, out, group_offsets=offsets, stream=stream)
