"""The Python face of the native kernels: each function takes CUDA tensors, checks what the
kernel cannot check itself, and launches on the current stream. Nothing here computes in
PyTorch, and nothing falls back: without a GPU or the compiled libraries it raises
``KernelError``.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build
from .errors import KernelError

F32, BF16 = 0, 1
EPI_STORE, EPI_ADD, EPI_SWIGLU, EPI_SWIGLU_PAIRS = 0, 1, 2, 3
PAGE = 64  # positions per cache page (MB_PAGE in csrc/common.cuh)

_c = ctypes
_vp, _i, _f, _d, _ll = _c.c_void_p, _c.c_int, _c.c_float, _c.c_double, _c.c_longlong


def code_of(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"tensors of {dtype} are not supported by the kernels")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a kernel was given a tensor that is not on the GPU")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream of the current device as the integer that the kernels take."""
    if _raw_stream is not None:                     # the short way (no Stream object)
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def require_gpu() -> None:
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this library computes on a B200 only (no CPU path)")
    major, minor = torch.cuda.get_device_capability()
    if major != 10:
        raise KernelError(f"the kernels are built for sm_100a; this device is sm_{major}{minor}")


class Launches:
    """How many kernels of this library were launched (a graph replay counts the kernels that
    were captured into it)."""
    count = 0


CLASS_OF = {"mb_gemm_tc": "products", "mb_gemm_simt": "products",
            "mb_attention_simt": "attention", "mb_attention_decode": "attention",
            "mb_attention_decode_clusters": "attention", "mb_attention_prefill": "attention",
            "mb_attention_prefill_tc": "attention", "mb_rmsnorm": "norms",
            "mb_qk_norm_rope_store": "rotary", "mb_embed": "embedding", "mb_swiglu": "activation",
            "mb_argmax": "sampling", "mb_sample": "sampling", "mb_sample_filtered": "sampling",
            "mb_advance_decode": "sampling", "mb_dynamic_tanh": "norms",
            "mb_gated_act": "activation", "mb_scale": "activation", "mb_add_bias": "activation",
            "mb_gemm_tc_gated": "products", "mb_latent_prep": "rotary",
            "mb_heads_gemm": "products", "mb_latent_attention": "attention",
            "mb_latent_attention_mma": "attention",
            "mb_moe_route": "routing", "mb_moe_plan": "routing", "mb_moe_route_plan": "routing", "mb_moe_gemm": "products",
            "mb_moe_combine": "routing", "mb_stream_step": "norms", "mb_add_scaled": "norms",
            "mb_token_shift": "recurrence", "mb_wkv_scan": "recurrence",
            "mb_mlstm_scan": "recurrence", "mb_tanh": "recurrence",
            "mb_retention_scan": "recurrence", "mb_retention_chunked": "recurrence",
            "mb_norm_add": "norms", "mb_cast_rows": "norms",
            "mb_unary_act": "activation", "mb_softcap": "activation",
            "mb_pass_input": "embedding", "mb_wide_qk_norm": "rotary",
            "mb_short_conv": "recurrence", "mb_linear_state_scan": "recurrence"}


class Timing:
    """Times every kernel call by its class while it is open (CUDA events around each call,
    which also keeps a kernel from starting under the tail of the one before: a diagnosis, not
    the speed of the product path). The role of the reference's ``TTimedBackend``
    (``demos/infer/llm-bench.lpr:58-236``).

        with Timing() as t:
            engine.step(...)
        t.shares()   # {"products": ms, "attention": ms, ...}, after a synchronize

    The time between the end of one call and the start of the next (the host preparing the
    next launch, other work on the stream) is booked as ``between``, so that the classes add
    up to the time from the first call to the last.
    """
    current: Optional["Timing"] = None

    def __init__(self):
        self.events = []

    def __enter__(self):
        Timing.current = self
        return self

    def __exit__(self, *exc):
        Timing.current = None

    def shares(self, start=None, end=None) -> dict:
        """``start``, ``end``: events recorded before the first and after the last call, whose
        distance to them is booked as ``between`` too."""
        torch.cuda.synchronize()
        out: dict = {}
        last = start
        for name, e0, e1 in self.events:
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
            if last is not None:
                out["between"] = out.get("between", 0.0) + last.elapsed_time(e0)
            last = e1
        if end is not None and last is not None:
            out["between"] = out.get("between", 0.0) + last.elapsed_time(end)
        return out


def read_trace() -> list:
    """The kernels' own timeline, from a build with ``MORMOT_B200_NVCC_FLAGS=-DMB_TRACE``: every
    CTA of the decode kernels (matrix products, RMSNorm, q/k norm + rotary, decode attention)
    leaves its start and end on the GPU's nanosecond timer. Returns ``[(start_ns, end_ns,
    kind)]`` of all CTAs since the last call, sorted by start (``kind``: "product", "norm",
    "rotary", "attention"); empty in an ordinary build. Unlike ``Timing`` this does not change
    the schedule: it shows a step as it runs inside a CUDA graph, kernels overlapping where
    programmatic dependent launch lets them."""
    names = {1: "product", 2: "norm", 3: "rotary", 4: "attention"}
    rows = []
    cap = 1 << 17
    buf = (_c.c_ulonglong * (2 * cap))()
    for lib in ("gemm_tc", "elementwise", "rope", "attention_mma"):
        handle = build.load_library(lib)
        if not hasattr(handle, "mb_trace_read"):
            continue
        n = handle.mb_trace_read(buf, cap)
        mask = (1 << 56) - 1
        rows += [(buf[2 * i] & mask, buf[2 * i + 1] & mask, names.get(buf[2 * i] >> 56, "?"))
                 for i in range(n)]
    rows.sort()
    return rows


def _call(libname: str, fn: str, argtypes, *args, launches: int = 1) -> None:
    lib = build.load_library(libname)
    f = getattr(lib, fn)
    if f.argtypes is None:
        f.argtypes = argtypes
        f.restype = _i
    timing = Timing.current
    if timing is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    rc = f(*args)
    if rc != 0:
        raise KernelError(lib.mb_last_error().decode(errors="replace"))
    if timing is not None:
        e1.record()
        timing.events.append((CLASS_OF.get(fn, "other"), e0, e1))
    Launches.count += launches


def _contig(t: torch.Tensor, what: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{what} is not contiguous")


# ------------------------------------------------------------------------------ elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, x: torch.Tensor, scale: float = 1.0) -> None:
    """x[t, :] = table[ids[t], :] * scale as float32; x [T, H], or [S, T, H]: S residual
    streams that all start as the same rows."""
    copies = x.shape[0] if x.dim() == 3 else 1
    T, H = x.shape[-2:]
    _contig(table, "the embedding"), _contig(x, "x")
    assert ids.dtype == torch.int32 and x.dtype == torch.float32 and table.shape[1] == H
    _call("elementwise", "mb_embed", [_vp, _i, _vp, _vp, _i, _i, _i, _f, _i, _ll, _vp],
          _ptr(table), code_of(table.dtype), _ptr(ids), _ptr(x), T, H, table.shape[0],
          float(scale), copies, T * H, _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor],
            rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
            partial: Optional[torch.Tensor] = None) -> None:
    """out[r] = w * x[rows[r] or r] / rms(x). ``partial`` [parts, T, H] float32 is first added
    into x (the split results of the matrix product before)."""
    H = x.shape[-1]
    R = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
    assert x.dtype == torch.float32 and w.numel() == H
    _contig(x, "x")
    parts, stride = 0, 0
    if partial is not None:
        assert partial.dtype == torch.float32 and partial.is_contiguous()
        parts, stride = partial.shape[0], partial.stride(0)
    _call("elementwise", "mb_rmsnorm",
          [_vp, _vp, _i, _ll, _vp, _i, _f, _vp, _i, _vp, _i, _i, _vp],
          _ptr(x), _ptr(partial), parts, stride, _ptr(w), code_of(w.dtype), float(eps),
          _ptr(out), code_of(out.dtype) if out is not None else F32, _ptr(rows), R, H, _stream())


def add_partials(x: torch.Tensor, partial: torch.Tensor) -> None:
    """x += partial[0] + partial[1] + ... (float32 [parts, T, H]), in that order."""
    assert x.dtype == torch.float32 and partial.dtype == torch.float32 and partial.is_contiguous()
    _contig(x, "x")
    T, H = x.shape
    _call("elementwise", "mb_rmsnorm",
          [_vp, _vp, _i, _ll, _vp, _i, _f, _vp, _i, _vp, _i, _i, _vp],
          _ptr(x), _ptr(partial), partial.shape[0], partial.stride(0), None, F32, 0.0, None, F32,
          None, T, H, _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[T, I] = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.dtype == out.dtype
    _contig(gate_up, "gate_up"), _contig(out, "out")
    _call("elementwise", "mb_swiglu", [_vp, _vp, _i, _i, _i, _vp],
          _ptr(gate_up), _ptr(out), code_of(out.dtype), T, I, _stream())


def qk_norm_rope_store(qkv, q_norm, k_norm, eps, inv_freq, rot_dim, step, line, nh, nkv, hd,
                       write_kv: bool, partial: Optional[torch.Tensor] = None,
                       q_out: Optional[torch.Tensor] = None, vd: int = 0,
                       unit_after: bool = False) -> None:
    """Per-head norm of q and k, rotary positions, q in place (or into ``q_out``), k and v into
    the cache line. ``partial`` [parts, T, width] float32: the split sums of the q/k/v product,
    which stand for ``qkv`` (then None) and are added up here. A row may hold more columns
    behind q, k and v (another projection of the same product); they are left alone.
    ``unit_after``: q and k are divided by their root mean square after the rotation, without
    a weight, instead of the weighted norm before it."""
    if partial is not None:
        assert partial.dtype == torch.float32 and partial.is_contiguous() and q_out is not None
        T, width = partial.shape[1], partial.shape[2]
        dtype_code = code_of(q_out.dtype)
    else:
        T, width = qkv.shape
        _contig(qkv, "qkv")
        dtype_code = code_of(qkv.dtype)
    vd = vd or hd
    assert width >= (nh + nkv) * hd + nkv * vd
    if rot_dim > 0 and inv_freq is None:
        raise KernelError("a rotary encoding without its frequencies (is the position "
                          "encoding bound?)")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() < rot_dim // 2):
        raise KernelError(f"{inv_freq.numel()} frequencies for {rot_dim} rotating values")
    if (q_norm is None) != (k_norm is None):
        raise KernelError("q_norm and k_norm come together")
    wd = code_of(q_norm.dtype) if q_norm is not None else F32
    _call("rope", "mb_qk_norm_rope_store",
          [_vp, _vp, _i, _ll, _vp, _i, _vp, _vp, _i, _f, _vp, _i, _vp, _vp, _vp, _i, _i,
           _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
          _ptr(qkv), _ptr(partial), partial.shape[0] if partial is not None else 0,
          partial.stride(0) if partial is not None else 0, _ptr(q_out), dtype_code,
          _ptr(q_norm), _ptr(k_norm), wd, float(eps),
          _ptr(inv_freq), rot_dim, _ptr(step.tok_slot), _ptr(step.tok_pos),
          _ptr(line.page_table), line.max_pages, line.ring_pages, _ptr(line.k), _ptr(line.v),
          T, nh, nkv, hd, 1 if write_kv else 0, vd, width, 1 if unit_after else 0, _stream())


# "clamped_swish": g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(1.702 g') (u' + 1)
ACT_SILU, ACT_GELU_TANH, ACT_CLAMPED_SWISH, ACT_RELU_SQUARED = 0, 1, 2, 3
ACTIVATIONS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH, "clamped_swish": ACT_CLAMPED_SWISH}
# activations of one input (a feed-forward without a gate): act(W_up h)
UNARY_ACTIVATIONS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH,
                     "relu_squared": ACT_RELU_SQUARED}


def dynamic_tanh(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor,
                 out: torch.Tensor, rows: Optional[torch.Tensor] = None,
                 n_rows: Optional[int] = None, partial: Optional[torch.Tensor] = None,
                 residual_bias: Optional[torch.Tensor] = None) -> None:
    """out[r] = tanh(alpha * x[rows[r] or r]) * w + b; ``alpha``: one float32 on the device.
    ``partial`` [parts, T, H] float32 is first added into x. ``residual_bias`` [H] is added
    into x after out was formed (the bias of a product that is accumulated onto x later)."""
    H = x.shape[-1]
    R = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
    assert x.dtype == torch.float32 and w.numel() == H and b.numel() == H
    assert alpha.dtype == torch.float32 and w.dtype == b.dtype
    _contig(x, "x")
    parts, stride = 0, 0
    if partial is not None:
        assert partial.dtype == torch.float32 and partial.is_contiguous()
        parts, stride = partial.shape[0], partial.stride(0)
    if residual_bias is not None:
        assert residual_bias.dtype == w.dtype and residual_bias.numel() == H
    _call("elementwise", "mb_dynamic_tanh",
          [_vp, _vp, _i, _ll, _vp, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _vp, _vp],
          _ptr(x), _ptr(partial), parts, stride, _ptr(w), _ptr(b), code_of(w.dtype), _ptr(alpha),
          _ptr(out), code_of(out.dtype), _ptr(rows), R, H, _ptr(residual_bias), _stream())


def add_bias(x: torch.Tensor, b: torch.Tensor) -> None:
    """x[t, :] += b (x float32)."""
    assert x.dtype == torch.float32 and b.numel() == x.shape[1]
    _contig(x, "x")
    _call("elementwise", "mb_add_bias", [_vp, _vp, _i, _i, _i, _vp],
          _ptr(x), _ptr(b), code_of(b.dtype), x.shape[0], x.shape[1], _stream())


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, act: int,
              gate_bias: Optional[torch.Tensor] = None, up_bias: Optional[torch.Tensor] = None,
              x: Optional[torch.Tensor] = None, x_bias: Optional[torch.Tensor] = None,
              limit: float = 0.0) -> None:
    """out[T, I] = act(gate_up[:, :I] + gate_bias) * (gate_up[:, I:] + up_bias); with ``x`` and
    ``x_bias`` the float32 residual rows also receive that bias (the one of the product that
    is added onto them next)."""
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.dtype == out.dtype
    _contig(gate_up, "gate_up"), _contig(out, "out")
    biases = [b for b in (gate_bias, up_bias, x_bias) if b is not None]
    assert all(b.dtype == biases[0].dtype for b in biases)
    if x is not None:
        assert x.dtype == torch.float32 and x.is_contiguous() and x_bias.numel() == x.shape[1]
    _call("elementwise", "mb_gated_act",
          [_vp, _vp, _i, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _i, _f, _vp],
          _ptr(gate_up), _ptr(out), code_of(out.dtype), T, I, act, _ptr(gate_bias),
          _ptr(up_bias), code_of(biases[0].dtype) if biases else F32, _ptr(x), _ptr(x_bias),
          x.shape[1] if x is not None else 0, float(limit), _stream())


def norm_add(y: torch.Tensor, w: torch.Tensor, eps: float, x: torch.Tensor,
             h: Optional[torch.Tensor] = None) -> None:
    """x += w * y / rms(y), row by row (float32); ``y`` [T, H] float32 or the split sums
    [parts, T, H] of a product, added up here in split order. ``h`` [T, H] (activation type):
    receives the new x rounded, for the sublayer that reads the residual next."""
    T, H = x.shape
    assert x.dtype == torch.float32 and y.dtype == torch.float32 and w.numel() == H
    _contig(x, "x"), _contig(y, "y")
    parts, stride = (1, 0) if y.dim() == 2 else (y.shape[0], y.stride(0))
    assert y.shape[-2:] == (T, H)
    if h is not None:
        assert h.shape == (T, H) and h.is_contiguous()
    _call("elementwise", "mb_norm_add", [_vp, _i, _ll, _vp, _i, _f, _vp, _vp, _i, _i, _i, _vp],
          _ptr(y), parts, stride, _ptr(w), code_of(w.dtype), float(eps), _ptr(x), _ptr(h),
          code_of(h.dtype) if h is not None else F32, T, H, _stream())


def cast_rows(x: torch.Tensor, h: torch.Tensor) -> None:
    """h = x (float32) rounded to h's type."""
    assert x.dtype == torch.float32 and x.shape == h.shape
    _contig(x, "x"), _contig(h, "h")
    _call("elementwise", "mb_cast_rows", [_vp, _vp, _i, _ll, _vp], _ptr(x), _ptr(h),
          code_of(h.dtype), x.numel(), _stream())


def unary_act(z: torch.Tensor, out: torch.Tensor, act: int,
              table: Optional[torch.Tensor] = None, col0: int = 0,
              ids: Optional[torch.Tensor] = None) -> None:
    """out[t, c] = act(z[t, c]); with ``table`` [V, >= col0 + N] and ``ids`` int32 [T] also
    times table[ids[t], col0 + c] (a factor that the token itself brings)."""
    T, N = out.shape
    assert z.shape == (T, N) and z.dtype == out.dtype and z.stride(1) == 1
    _contig(out, "out")
    if table is not None:
        assert ids is not None and ids.dtype == torch.int32 and ids.numel() == T
        assert table.dim() == 2 and table.stride(1) == 1 and table.shape[1] >= col0 + N
    _call("elementwise", "mb_unary_act",
          [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _vp],
          _ptr(z), z.stride(0), _ptr(out), code_of(out.dtype), T, N, act, _ptr(table),
          code_of(table.dtype) if table is not None else F32,
          table.stride(0) if table is not None else 0, col0, _ptr(ids),
          table.shape[0] if table is not None else 0, _stream())


def softcap_rows(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap) (float32, contiguous)."""
    assert x.dtype == torch.float32
    _contig(x, "x")
    _call("elementwise", "mb_softcap", [_vp, _ll, _f, _vp], _ptr(x), x.numel(), float(cap),
          _stream())


def scale_rows(x: torch.Tensor, factor: float) -> None:
    """x *= factor (float32, contiguous)."""
    assert x.dtype == torch.float32
    _contig(x, "x")
    _call("elementwise", "mb_scale", [_vp, _ll, _f, _vp], _ptr(x), x.numel(), float(factor),
          _stream())


def pass_input(x: torch.Tensor, b: torch.Tensor, x0: Optional[torch.Tensor] = None) -> None:
    """x[t, :] += x0[t, :] + b (x, x0 float32 [T, H]; b [H]): what a pass through looped layers
    starts from."""
    assert x.dtype == torch.float32 and b.numel() == x.shape[1] and b.is_contiguous()
    _contig(x, "x")
    if x0 is not None:
        assert x0.dtype == torch.float32 and x0.shape == x.shape and x0.is_contiguous()
    _call("elementwise", "mb_pass_input", [_vp, _vp, _vp, _i, _i, _i, _vp],
          _ptr(x), _ptr(x0), _ptr(b), code_of(b.dtype), x.shape[0], x.shape[1], _stream())


def wide_qk_norm(qkv: torch.Tensor, qw: int, kw: int, wq: torch.Tensor, wk: torch.Tensor,
                 eps: float, copy_k: bool) -> None:
    """Rows [q (qw) | k (kw) | ...]: q and k are each normed over their whole width with the
    weights ``wq`` [qw] and ``wk`` [kw], in place; ``copy_k``: the k values as they came are
    first copied into the kw columns behind k (without weights nothing else happens)."""
    T, ld = qkv.shape
    _contig(qkv, "qkv")
    assert (wq is None and wk is None and copy_k) or (
        wq.numel() == qw and wk.numel() == kw and wq.dtype == wk.dtype)
    assert ld >= qw + kw * (2 if copy_k else 1)
    _call("elementwise", "mb_wide_qk_norm", [_vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _f, _i, _vp],
          _ptr(qkv), code_of(qkv.dtype), ld, T, qw, kw, _ptr(wq), _ptr(wk),
          code_of(wq.dtype) if wq is not None else F32,
          float(eps), 1 if copy_k else 0, _stream())


# ------------------------------------------------------------------------------ residual streams
def _terms(terms):
    """[(y [T, H] float32, factor)] as the arrays the kernels take."""
    n = len(terms)
    ys = (_vp * n)(*[_ptr(y) for y, _ in terms])
    fs = (_f * n)(*[float(f) for _, f in terms])
    for y, _ in terms:
        assert y.dtype == torch.float32 and y.is_contiguous()
    return ys, fs, n


def stream_step(x: torch.Tensor, update=None, read=None) -> None:
    """One pass over the residual streams x [S, T, H] (or [T, H]: one stream), float32.
    ``update = (mix [S, S], out [S], terms)``: x_t <- sum_s mix[s, t] x_s + out[t] y with
    y = sum_b factor_b y_b over ``terms = [(y_b, factor_b)]``. ``read = (in [S] or None (ones),
    w [H], eps, out [R, H], rows int32 [R] or None, R)``: the layer norm of u = sum_s in[s] x_s
    (after the update) times w."""
    S = x.shape[0] if x.dim() == 3 else 1
    T, H = x.shape[-2:]
    _contig(x, "x")
    assert x.dtype == torch.float32
    mix = outc = ys = fs = None
    n = 0
    if update is not None:
        mix, outc, terms = update
        assert mix.dtype == outc.dtype == torch.float32 and mix.numel() == S * S
        assert outc.numel() == S and mix.is_contiguous()
        ys, fs, n = _terms(terms)
        for y, _ in terms:
            assert y.shape == (T, H)
    a = w = out = rows = None
    eps, R = 0.0, T
    if read is not None:
        a, w, eps, out, rows, R = read
        assert a is None or (a.dtype == torch.float32 and a.numel() == S)
        assert w.numel() == H and out.is_contiguous() and out.shape == (R, H)
    _call("streams", "mb_stream_step",
          [_vp, _ll, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _f, _vp, _i, _vp, _i, _i, _vp],
          _ptr(x), T * H, S, _ptr(mix), _ptr(outc), ys, fs, n, _ptr(a), _ptr(w),
          code_of(w.dtype) if w is not None else F32, float(eps), _ptr(out),
          code_of(out.dtype) if out is not None else F32, _ptr(rows), R, H, _stream())


def add_scaled(x: torch.Tensor, terms, store: bool = False) -> None:
    """x (+)= sum_b factor_b y_b for ``terms = [(y_b, factor_b)]``, all float32 of x's shape."""
    assert x.dtype == torch.float32
    _contig(x, "x")
    ys, fs, n = _terms(terms)
    for y, _ in terms:
        assert y.shape == x.shape
    _call("streams", "mb_add_scaled", [_vp, _vp, _vp, _i, _ll, _i, _vp],
          _ptr(x), ys, fs, n, x.numel(), 1 if store else 0, _stream())


# ------------------------------------------------------------------------------ recurrences
def token_shift(h: torch.Tensor, state: torch.Tensor, step, out: torch.Tensor) -> None:
    """out[t] = [h[t] ; h[t-1] - h[t]]; the row before a sequence's first row of this step is
    read from its state (``state`` [slots, >= W] float32, a view whose rows may lie apart)."""
    T, W = h.shape
    _contig(h, "h"), _contig(out, "out")
    assert out.shape == (T, 2 * W) and out.dtype == h.dtype
    assert state.dtype == torch.float32 and state.stride(1) == 1 and state.shape[1] >= W
    _call("recurrent", "mb_token_shift",
          [_vp, _i, _vp, _ll, _ll, _vp, _vp, _vp, _vp, _i, _i, _vp],
          _ptr(h), code_of(h.dtype), _ptr(state), state.stride(0), 0, _ptr(step.tok_seq),
          _ptr(step.seq_start), _ptr(step.seq_slot), _ptr(out), T, W, _stream())


def tanh_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = tanh(x): float32 rows in (they may lie apart), the activation type out."""
    assert x.dtype == torch.float32 and x.stride(1) == 1 and out.is_contiguous()
    assert x.shape == out.shape
    _call("recurrent", "mb_tanh", [_vp, _i, _vp, _i, _i, _i, _vp], _ptr(x), x.stride(0),
          _ptr(out), code_of(out.dtype), x.shape[0], x.shape[1], _stream())


def wkv_scan(r, k, v, lw, g, w0, u, normw, eps: float, state: torch.Tensor,
             h: torch.Tensor, step, out: torch.Tensor, heads: int, dim: int) -> None:
    """The decaying matrix state, token after token (csrc/recurrent.cu). r, k, v, lw, g:
    float32 [T, >= heads * dim] with one row stride; the state row of a slot holds the last h
    (``h.shape[1]`` values) and then heads x dim x dim values."""
    T = out.shape[0]
    state_off = 0
    ld = r.stride(0)
    for t in (r, k, v, lw, g):
        assert t.dtype == torch.float32 and t.stride(1) == 1 and t.stride(0) == ld
    for t in (w0, u, normw):
        assert t.dtype == torch.float32 and t.numel() == heads * dim and t.is_contiguous()
    _contig(out, "out"), _contig(h, "h")
    assert out.dtype == h.dtype and out.shape == (T, heads * dim) and state.dtype == torch.float32
    assert state.stride(1) == 1 and state.shape[1] >= h.shape[1] + heads * dim * dim
    # where a step has few (sequence, head) pairs a head's columns are dealt over several
    # blocks, which leave their outputs here for the kernel that norms and gates them
    raw = torch.empty((T, heads * dim), dtype=torch.float32, device=out.device)
    _call("recurrent", "mb_wkv_scan",
          [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _f, _vp, _ll, _ll, _vp, _i, _i, _vp, _vp,
           _vp, _vp, _i, _i, _i, _i, _vp],
          _ptr(r), _ptr(k), _ptr(v), _ptr(lw), _ptr(g), ld, _ptr(w0), _ptr(u), _ptr(normw),
          float(eps), _ptr(state), state.stride(0), state_off, _ptr(h), code_of(h.dtype),
          h.shape[1], _ptr(step.seq_start), _ptr(step.seq_slot), _ptr(out), _ptr(raw), T, step.B,
          heads, dim, _stream(), launches=1 if step.B * heads >= 96 else 2)


def mlstm_scan(z: torch.Tensor, cols, bi, bf, cap: float, q_scale: float, normw, eps: float,
               state: torch.Tensor, step, out: torch.Tensor, heads: int,
               dim: int, vdim: int) -> None:
    """The gated matrix memory, token after token (csrc/recurrent.cu). z: the fused projection
    [T, ld] float32; ``cols`` = the first columns of q, k, v, the output gate, the input gate
    and the forget gate in it. The state row of a slot holds, per head, dim x vdim values of
    the memory, dim of the normalizer and the running maximum."""
    T = out.shape[0]
    state_off = 0
    assert z.dtype == torch.float32 and z.stride(1) == 1 and len(cols) == 6
    for t in (bi, bf):
        assert t.dtype == torch.float32 and t.numel() == heads
    assert normw.dtype == torch.float32 and normw.numel() == heads * vdim
    _contig(out, "out")
    assert out.shape == (T, heads * vdim) and state.dtype == torch.float32
    assert state.stride(1) == 1 and state.shape[1] >= heads * (dim * vdim + dim + 1)
    raw = torch.empty((T, heads * vdim), dtype=torch.float32, device=out.device)   # as in wkv_scan
    _call("recurrent", "mb_mlstm_scan",
          [_vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _f, _f, _vp, _f, _vp, _ll, _ll, _vp, _vp,
           _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
          _ptr(z), z.stride(0), *[int(c) for c in cols], _ptr(bi), _ptr(bf), float(cap),
          float(q_scale), _ptr(normw), float(eps), _ptr(state), state.stride(0), state_off,
          _ptr(step.seq_start), _ptr(step.seq_slot), _ptr(out), _ptr(raw), code_of(out.dtype), T,
          step.B, heads, dim, vdim, _stream(), launches=1 if step.B * heads >= 96 else 2)


def retention_chunk(dim: int, vdim: int) -> int:
    """The chunk in which ``retention_scan`` walks a long portion of heads of dim x vdim values
    (0: such heads are only walked token by token): what mb_retention_chunk of
    csrc/recurrent.cu computes, from what a block stages in shared memory."""
    def need(c):
        return 4 * (2 * dim * (c + 4) + c * (c + 4) + 2 * c * ((vdim + 3) // 4 * 4))
    return 64 if need(64) <= 112 * 1024 else 32 if need(32) <= 200 * 1024 else 0


def retention_scan(z: torch.Tensor, cols, decay: torch.Tensor, k_scale: float,
                   inv_freq: Optional[torch.Tensor], rot_dim: int, eps: float,
                   state: torch.Tensor, step, out: torch.Tensor, heads: int, dim: int,
                   vdim: int, chunked: Optional[bool] = None) -> None:
    """Retention (csrc/recurrent.cu). z: the fused projection [T, ld] float32; ``cols`` = the
    first columns of q, k, v and the output gate in it; ``decay`` float32 [heads] on the
    device. The state row of a slot holds heads x dim x vdim values. A step of at least 128
    tokens and two or more a sequence is walked chunk by chunk (every chunk's own sum, the
    walk over the chunks' states, every chunk's outputs: three kernels that fill the device),
    any other token by token; ``chunked`` forces one form. The choice depends on the step's
    shape only, so a captured launch stays valid."""
    T = out.shape[0]
    assert z.dtype == torch.float32 and z.stride(1) == 1 and len(cols) == 4
    assert decay.dtype == torch.float32 and decay.numel() == heads
    if rot_dim > 0 and (inv_freq is None or inv_freq.dtype != torch.float32
                        or inv_freq.numel() < rot_dim // 2):
        raise KernelError(f"a rotation of {rot_dim} values without its frequencies")
    _contig(out, "out")
    assert out.shape == (T, heads * vdim) and state.dtype == torch.float32
    assert state.stride(1) == 1 and state.shape[1] >= heads * dim * vdim
    if chunked is None:
        chunked = T >= 128 and T >= 2 * step.B
    C = retention_chunk(dim, vdim) if chunked else 0
    if C:
        chunks = (T + C - 1) // C + step.B
        W = torch.empty((chunks, heads, dim, (vdim + 3) // 4 * 4), dtype=torch.float32,
                        device=out.device)
        _call("recurrent", "mb_retention_chunked",
              [_vp, _i, _i, _i, _i, _i, _vp, _f, _vp, _i, _vp, _f, _vp, _ll, _ll, _vp, _vp, _vp,
               _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
              _ptr(z), z.stride(0), *[int(c) for c in cols], _ptr(decay), float(k_scale),
              _ptr(inv_freq), rot_dim, _ptr(step.tok_pos), float(eps), _ptr(state),
              state.stride(0), 0, _ptr(step.seq_start), _ptr(step.seq_slot), _ptr(out), _ptr(W),
              chunks, code_of(out.dtype), T, step.B, heads, dim, vdim, _stream(), launches=3)
        return
    raw = torch.empty((T, heads * vdim), dtype=torch.float32, device=out.device)   # as in wkv_scan
    _call("recurrent", "mb_retention_scan",
          [_vp, _i, _i, _i, _i, _i, _vp, _f, _vp, _i, _vp, _f, _vp, _ll, _ll, _vp, _vp, _vp, _vp,
           _i, _i, _i, _i, _i, _i, _vp],
          _ptr(z), z.stride(0), *[int(c) for c in cols], _ptr(decay), float(k_scale),
          _ptr(inv_freq), rot_dim, _ptr(step.tok_pos), float(eps), _ptr(state), state.stride(0),
          0, _ptr(step.seq_start), _ptr(step.seq_slot), _ptr(out), _ptr(raw),
          code_of(out.dtype), T, step.B, heads, dim, vdim, _stream(),
          launches=1 if step.B * heads >= 96 else 2)


def short_conv(z: torch.Tensor, col0: int, w: torch.Tensor, state: torch.Tensor, step,
               out: torch.Tensor) -> None:
    """out[t, c] = silu(sum_j w[c, j] * z[t - taps + 1 + j, col0 + c]) within each sequence;
    the inputs before a step's first token come from ``state`` ([slots, >= (taps - 1) * C]
    float32, a view whose rows may lie apart: zeros when a sequence starts), which afterwards
    holds the step's last taps - 1 inputs (csrc/linear_state.cu)."""
    T = z.shape[0]
    C, taps = w.shape
    assert z.dtype == torch.float32 and z.stride(1) == 1 and z.shape[1] >= col0 + C
    assert w.dtype == torch.float32 and w.is_contiguous()
    assert out.dtype == torch.float32 and out.shape == (T, C) and out.is_contiguous()
    assert state.dtype == torch.float32 and state.stride(1) == 1
    assert state.shape[1] >= (taps - 1) * C
    _call("linear_state", "mb_short_conv",
          [_vp, _i, _i, _vp, _i, _i, _vp, _ll, _ll, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
          _ptr(z), z.stride(0), col0, _ptr(w), taps, C, _ptr(state), state.stride(0), 0,
          _ptr(step.tok_seq), _ptr(step.seq_start), _ptr(step.seq_slot), _ptr(out),
          out.stride(0), T, step.B, _stream(), launches=2 if taps > 1 else 1)


def linear_state_scan(mode: str, qkv: torch.Tensor, cols, group: int, gate: torch.Tensor,
                      gate_col: int, normw: torch.Tensor, eps: float, state: torch.Tensor, step,
                      out: torch.Tensor, heads: int, dim: int, vdim: int,
                      decay_logits: Optional[torch.Tensor] = None, decay_col: int = 0,
                      decay_bias: Optional[torch.Tensor] = None, inv_tau: float = 1.0,
                      scalars: Optional[torch.Tensor] = None, beta_col: int = 0,
                      rate_col: int = 0, a_log: Optional[torch.Tensor] = None,
                      dt_bias: Optional[torch.Tensor] = None, unit_eps: float = 0.0) -> None:
    """A matrix state per head walked token by token (csrc/linear_state.cu). ``qkv`` float32
    [T, ld] with ``cols`` = the first columns of q, k and v in it; ``group`` heads share one q
    and k. ``mode`` "gla": S <- diag(a) S + k v^T with a = sigmoid(decay_logits + decay_bias)
    ^ inv_tau per key channel and q scaled by dim^(-1/2). ``mode`` "delta": q and k brought
    to unit length (``unit_eps`` under the root; q also times dim^(-1/2)), S <- g S,
    u = beta (v - S^T k), S <- S + k u^T with beta = sigmoid(scalars[beta_col + h]) and
    g = exp(-exp(a_log[h]) softplus(scalars[rate_col + h] + dt_bias[h])). Then o = S^T q over its
    root mean square, times ``normw`` [vdim], times silu(gate). The state row of a slot holds
    heads x dim x vdim values."""
    T = out.shape[0]
    f32 = torch.float32
    assert mode in ("gla", "delta") and len(cols) == 3
    assert qkv.dtype == f32 and qkv.stride(1) == 1 and gate.dtype == f32 and gate.stride(1) == 1
    assert normw.dtype == f32 and normw.numel() == vdim
    _contig(out, "out")
    assert out.shape == (T, heads * vdim) and state.dtype == f32 and state.stride(1) == 1
    assert state.shape[1] >= heads * dim * vdim
    if mode == "gla":
        assert decay_logits.dtype == f32 and decay_logits.stride(1) == 1
        assert decay_bias.dtype == f32 and decay_bias.numel() == heads * dim
    else:
        assert scalars.dtype == f32 and scalars.stride(1) == 1
        assert a_log.dtype == f32 and a_log.numel() == heads
        assert dt_bias.dtype == f32 and dt_bias.numel() == heads
    # where a step has few (sequence, head) pairs a head's columns are dealt over several
    # blocks, which leave their outputs here for the kernel that norms and gates them
    sliced = step.B * heads < 96 and vdim > 32
    raw = torch.empty((T, heads * vdim), dtype=f32, device=out.device)
    _call("linear_state", "mb_linear_state_scan",
          [_i, _vp, _i, _i, _i, _i, _i, _vp, _i, _i, _vp, _f, _vp, _i, _i, _i, _vp, _vp, _f,
           _vp, _i, _i, _vp, _f, _vp, _ll, _ll, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
          0 if mode == "gla" else 1, _ptr(qkv), qkv.stride(0), *[int(c) for c in cols],
          int(group), _ptr(decay_logits),
          decay_logits.stride(0) if decay_logits is not None else 0, int(decay_col),
          _ptr(decay_bias), float(inv_tau), _ptr(scalars),
          scalars.stride(0) if scalars is not None else 0, int(beta_col), int(rate_col),
          _ptr(a_log), _ptr(dt_bias), float(unit_eps), _ptr(gate), gate.stride(0), int(gate_col),
          _ptr(normw), float(eps), _ptr(state), state.stride(0), 0, _ptr(step.seq_start),
          _ptr(step.seq_slot), _ptr(out), _ptr(raw), code_of(out.dtype), T, step.B, step.max_new,
          heads, dim, vdim, _stream(), launches=2 if sliced else 1)


# ------------------------------------------------------------------------------ latent attention
def latent_prep(f: Optional[torch.Tensor], q_col: int, kv_col: int, q_rank: int, kv_rank: int,
                rot_dim: int, w_q: torch.Tensor, w_kv: torch.Tensor, eps: float,
                inv_freq: Optional[torch.Tensor], rot_dims: int, amplitude: float, step, line,
                cq_out: torch.Tensor, write_cache: bool, partial: Optional[torch.Tensor] = None,
                gate_out: Optional[torch.Tensor] = None, gate_col: int = 0) -> None:
    """From the rows of ``f`` [T, ld]: the normed query latent into ``cq_out`` [T, q_rank] and
    the cache row [normed key/value latent ; rotated shared key part] of every token.
    ``partial`` [parts, T, ld] float32 stands for ``f`` (then None): the split sums of the
    product, added up here; the columns from ``gate_col`` on are then added up into
    ``gate_out`` [T, n] as well."""
    T = cq_out.shape[0]
    assert cq_out.is_contiguous() and cq_out.dtype == line.k.dtype
    assert w_q.dtype == w_kv.dtype
    assert line.head_dim == kv_rank + rot_dim and line.kv_heads == 1
    parts, stride, gate_n = 0, 0, 0
    if partial is not None:
        assert f is None and partial.dtype == torch.float32 and partial.is_contiguous()
        parts, stride, ld = partial.shape[0], partial.stride(0), partial.shape[2]
        if gate_out is not None:
            assert gate_out.is_contiguous() and gate_out.dtype == cq_out.dtype
            gate_n = gate_out.shape[1]
            assert gate_col + gate_n <= ld
    else:
        assert f.stride(1) == 1 and f.dtype == cq_out.dtype and gate_out is None
        ld = f.stride(0)
    _call("latent", "mb_latent_prep",
          [_vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _f, _vp, _i, _f, _vp, _vp, _vp, _i, _i,
           _vp, _vp, _i, _i, _vp, _i, _ll, _vp, _i, _i, _vp],
          _ptr(f), code_of(cq_out.dtype), ld, q_col, kv_col, q_rank, kv_rank, rot_dim,
          _ptr(w_q), _ptr(w_kv), code_of(w_q.dtype), float(eps), _ptr(inv_freq), rot_dims,
          float(amplitude), _ptr(step.tok_slot), _ptr(step.tok_pos), _ptr(line.page_table),
          line.max_pages, line.ring_pages, _ptr(line.k), _ptr(cq_out), T,
          1 if write_cache else 0, _ptr(partial), parts, stride, _ptr(gate_out), gate_col,
          gate_n, _stream())


def heads_gemm(a: torch.Tensor, lda_h: int, b: torch.Tensor, c: torch.Tensor, ldc_h: int,
               gate: Optional[torch.Tensor] = None, tail: int = 0, rot_dims: int = 0,
               inv_freq: Optional[torch.Tensor] = None, amplitude: float = 1.0,
               tok_pos: Optional[torch.Tensor] = None) -> None:
    """c[t, h*ldc_h + n] = sum_k a[t, h*lda_h + k] * b[h, n, k] for every head h (``b``
    [heads, N, K]). ``gate`` [T, >= heads*N]: c is multiplied by its sigmoid. ``tail``: that
    many values of a behind the K multiplied ones are rotated by the token's position
    (``rot_dims`` of them turn) and stored behind c's N columns."""
    heads, N, Kd = b.shape
    M = a.shape[0]
    assert a.stride(1) == 1 and c.stride(1) == 1 and a.dtype == c.dtype and c.shape[0] == M
    _contig(b, "the heads' weight")
    if gate is not None:
        assert gate.dtype == a.dtype and gate.stride(1) == 1
    _call("latent", "mb_heads_gemm",
          [_vp, _i, _i, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _f, _vp,
           _vp],
          _ptr(a), code_of(a.dtype), a.stride(0), lda_h, _ptr(b), code_of(b.dtype), _ptr(c),
          c.stride(0), ldc_h, M, N, Kd, heads, _ptr(gate),
          gate.stride(0) if gate is not None else 0, tail, rot_dims, _ptr(inv_freq),
          float(amplitude), _ptr(tok_pos), _stream())


def latent_attention(q: torch.Tensor, out: torch.Tensor, step, line, nh: int, kv_rank: int,
                     rot_dim: int, window: int, scale: float) -> None:
    """Causal attention of every head over the cache rows [latent ; shared rotated key part];
    q [T, nh * (kv_rank + rot_dim)], out [T, nh * kv_rank] (the weighted latents)."""
    T = out.shape[0]
    _contig(out, "out"), _contig(q, "q")
    assert q.dtype == out.dtype == line.k.dtype
    _call("latent", "mb_latent_attention",
          [_vp, _i, _vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp],
          _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(line.k), code_of(out.dtype),
          _ptr(line.page_table), line.max_pages, line.ring_pages, _ptr(step.tok_slot),
          _ptr(step.tok_pos), T, nh, kv_rank, rot_dim, window, float(scale), _stream())


def latent_attention_mma(q: torch.Tensor, out: torch.Tensor, step, line, nh: int, kv_rank: int,
                         rot_dim: int, window: int, scale: float, splits: int,
                         scratch: Optional[torch.Tensor],
                         tickets: Optional[torch.Tensor] = None) -> None:
    """``latent_attention`` on the tensor cores (bfloat16; kv_rank and kv_rank + rot_dim
    multiples of 16, kv_rank at most 512). ``splits`` > 1: the key tiles of a sequence are
    dealt out over that many blocks, whose partial results meet in ``scratch`` (float32);
    ``tickets``: int32 zeros, one per 64 (token, head) rows of the step, left zero."""
    T = out.shape[0]
    _contig(out, "out"), _contig(q, "q")
    assert q.dtype == out.dtype == line.k.dtype == torch.bfloat16
    tiles = sum(-(-n * nh // 64) for n in step.host_new)
    if splits > 1:
        assert tickets is not None and tickets.dtype == torch.int32 and tickets.numel() >= tiles
    _call("latent_mma", "mb_latent_attention_mma",
          [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i,
           _vp, _ll, _vp, _vp],
          _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(line.k), _ptr(line.page_table),
          line.max_pages, line.ring_pages, _ptr(step.seq_start), _ptr(step.seq_past),
          _ptr(step.seq_slot), step.B, T, tiles, nh, kv_rank, rot_dim, window, float(scale),
          splits, _ptr(scratch), scratch.numel() if scratch is not None else 0,
          _ptr(tickets), _stream())


# ------------------------------------------------------------------------------ routed experts
def _parts_of(z: torch.Tensor):
    """z [T, N] or [parts, T, N] float32 (the split sums of a product): pointer arguments."""
    assert z.dtype == torch.float32 and z.stride(-1) == 1
    if z.dim() == 2:
        return 1, 0, z.stride(0)
    assert z.dim() == 3
    return z.shape[0], z.stride(0), z.stride(1)


ROUTE_SOFTMAX_OF_CHOSEN, ROUTE_SOFTMAX_OF_ALL = 0, 1


def moe_route(z: torch.Tensor, experts: int, top: int, shared_col: int, ids: torch.Tensor,
              w: torch.Tensor, sg: Optional[torch.Tensor], mode: int = 0,
              correction: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """Per row of z (float32 router logits, [T, N] or the split sums [parts, T, N] of the
    router's product): the ``top`` largest of the first ``experts`` columns into ``ids`` and
    the softmax over them into ``w``; ``sg`` = sigmoid of column ``shared_col``."""
    parts, stride, ldz = _parts_of(z)
    assert ids.dtype == torch.int32 and w.dtype == torch.float32
    assert correction is None or (correction.dtype == torch.float32
                                  and correction.numel() == experts)
    _call("moe", "mb_moe_route",
          [_vp, _i, _i, _ll, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _f, _vp],
          _ptr(z), ldz, parts, stride, experts, top, shared_col if sg is not None else -1,
          _ptr(ids), _ptr(w), _ptr(sg), z.shape[-2], mode, _ptr(correction), float(scale),
          _stream())


def moe_plan(ids: torch.Tensor, experts: int, bm: int, max_tiles: int,
             plan: torch.Tensor) -> None:
    assert plan.dtype == torch.int32 and plan.numel() >= 2 + experts + ids.numel() + 2 * max_tiles
    _call("moe", "mb_moe_plan", [_vp, _i, _i, _i, _i, _vp, _vp],
          _ptr(ids), ids.numel(), experts, bm, max_tiles, _ptr(plan), _stream())


def moe_route_plan(z: torch.Tensor, experts: int, top: int, shared_col: int, ids: torch.Tensor,
                   w: torch.Tensor, sg: Optional[torch.Tensor], bm: int, max_tiles: int,
                   plan: torch.Tensor, mode: int = 0, correction: Optional[torch.Tensor] = None,
                   scale: float = 1.0, routed: Optional[int] = None) -> None:
    """``moe_route`` and ``moe_plan`` as one kernel, for a step of at most 64 tokens.
    ``routed``: the columns that the router chooses among (``experts`` of them have lists;
    those after them are identity experts)."""
    parts, stride, ldz = _parts_of(z)
    assert ids.dtype == torch.int32 and w.dtype == torch.float32
    assert plan.dtype == torch.int32 and plan.numel() >= 2 + experts + ids.numel() + 2 * max_tiles
    _call("moe", "mb_moe_route_plan",
          [_vp, _i, _i, _ll, _i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp, _f, _i, _vp],
          _ptr(z), ldz, parts, stride, experts, top, shared_col if sg is not None else -1,
          _ptr(ids), _ptr(w), _ptr(sg), z.shape[-2], bm, max_tiles, _ptr(plan), mode,
          _ptr(correction), float(scale), routed if routed is not None else experts, _stream())


def moe_gemm(src: torch.Tensor, w: torch.Tensor, out: torch.Tensor, plan: torch.Tensor,
             assignments: int, max_tiles: int, bm: int, top: int, up: bool, act: int = ACT_SILU,
             weight: Optional[torch.Tensor] = None, limit: float = 0.0) -> None:
    """One of the experts' two products over the planned tiles. ``up``: w [E, 2N, K] (gate
    rows, then up rows), rows of ``src`` [T, K] gathered, out [A, N]. Else w [E, N, K], src
    [A, K], out [A, N] float32 at the assignment's own row, times ``weight`` [A]."""
    E = w.shape[0]
    N = w.shape[1] // (2 if up else 1)
    Kd = w.shape[2]
    _contig(src, "src"), _contig(out, "out"), _contig(w, "the experts' weight")
    assert src.shape[1] == Kd and out.shape[1] == N
    assert out.dtype == (src.dtype if up else torch.float32)
    _call("moe", "mb_moe_gemm",
          [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _f, _vp],
          _ptr(src), code_of(src.dtype), _ptr(w), code_of(w.dtype), _ptr(out), _ptr(plan),
          assignments, E, max_tiles, bm, top, N, Kd, 1 if up else 0, act, _ptr(weight),
          float(limit), _stream())


def moe_combine(x: torch.Tensor, y: torch.Tensor, top: int, shared: Optional[torch.Tensor],
                sg: Optional[torch.Tensor], ids: Optional[torch.Tensor] = None,
                w: Optional[torch.Tensor] = None, experts: int = 0,
                h: Optional[torch.Tensor] = None, store: bool = False) -> None:
    """x[t] += sum_k y[t*top + k] + sg[t] * shared[t] (all float32); ``shared`` [T, H] or the
    split sums [parts, T, H] of the shared expert's last product. With ``ids``: an assignment
    whose expert id is ``experts`` or more is an identity expert and adds w · h[t] instead of
    its row of y. ``store``: x = the sum."""
    T, H = x.shape
    assert x.dtype == y.dtype == torch.float32 and y.shape == (T * top, H)
    _contig(x, "x"), _contig(y, "y")
    parts, stride = 1, 0
    if shared is not None:
        assert shared.shape[-2:] == (T, H) and shared.is_contiguous()
        parts, stride, _ = _parts_of(shared)
    if ids is not None:
        assert ids.dtype == torch.int32 and w.dtype == torch.float32 and h.shape == (T, H)
        _contig(h, "h")
    _call("moe", "mb_moe_combine",
          [_vp, _vp, _i, _vp, _i, _ll, _vp, _i, _i, _vp, _vp, _i, _vp, _i, _i, _vp],
          _ptr(x), _ptr(y), top, _ptr(shared), parts, stride, _ptr(sg), T, H, _ptr(ids), _ptr(w),
          experts, _ptr(h), code_of(h.dtype) if h is not None else F32, 1 if store else 0,
          _stream())


# ------------------------------------------------------------------------------ products
def gemm_simt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """c = a · wᵀ (store), c += a · wᵀ (add, float32 c), or SwiGLU over w = [gate; up]
    (EPI_SWIGLU) or over a w whose rows alternate gate, up (EPI_SWIGLU_PAIRS)."""
    M, K = a.shape
    N = c.shape[1]
    assert w.shape[1] == K
    assert w.shape[0] == (2 * N if epilogue in (EPI_SWIGLU, EPI_SWIGLU_PAIRS) else N)
    assert c.shape[0] == M and a.stride(1) == 1 and c.stride(1) == 1
    _contig(w, "the weight")
    _call("gemm_simt", "mb_gemm_simt",
          [_vp, _i, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp],
          _ptr(a), code_of(a.dtype), a.stride(0), _ptr(w), code_of(w.dtype), _ptr(c),
          code_of(c.dtype), c.stride(0), M, N, K, epilogue, _stream())


# ------------------------------------------------------------------------------ attention
def attention_simt(q: torch.Tensor, q_stride: int, out: torch.Tensor, step, line, nh, nkv, hd,
                   window: int, scale: float, vd: int = 0,
                   sink: Optional[torch.Tensor] = None, softcap: float = 0.0,
                   gate: Optional[torch.Tensor] = None, gate_stride: int = 0,
                   slopes: Optional[torch.Tensor] = None, keep_first: int = 0) -> None:
    """``vd``: the size of a value row when it differs from ``hd``. ``sink``: float32 [nh],
    one more term exp(sink[h]) in the softmax denominators of head h. ``softcap`` > 0: scores
    become softcap * tanh(score / softcap). ``gate``: logits of q's type, head h of token t at
    ``gate[t * gate_stride + h]``; the head's output is multiplied by their sigmoid.
    ``slopes``: float32 [nh]; slopes[h] * (distance of key and query) is taken off head h's
    scores after the cap. ``keep_first``: with a window, the first so many positions of a
    sequence stay visible (the line must then keep all pages, not a ring)."""
    T = out.shape[0]
    _contig(out, "out")
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == nh)
    assert slopes is None or (slopes.dtype == torch.float32 and slopes.numel() == nh)
    assert gate is None or gate.dtype == out.dtype
    assert keep_first == 0 or line.ring_pages == 0
    _call("attention_simt", "mb_attention_simt",
          [_vp, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f,
           _i, _vp, _f, _vp, _i, _vp, _i, _vp],
          _ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(line.k), _ptr(line.v),
          code_of(out.dtype), _ptr(line.page_table), line.max_pages, line.ring_pages,
          _ptr(step.tok_seq), _ptr(step.tok_pos), _ptr(step.seq_slot), T, nh, nkv, hd,
          window, float(scale), vd or hd, _ptr(sink), float(softcap), _ptr(gate), gate_stride,
          _ptr(slopes), int(keep_first), _stream())


# ------------------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: torch.Tensor,
           scratch: Optional[torch.Tensor] = None) -> None:
    """out[r] = arg-max of row r; with ``scratch`` (8 bytes per row and 2048 values) wide rows
    are read by many CTAs."""
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    nbytes = scratch.numel() * scratch.element_size() if scratch is not None else 0
    _call("sampling", "mb_argmax", [_vp, _ll, _i, _i, _vp, _vp, _ll, _vp],
          _ptr(logits), logits.stride(0), rows, V, _ptr(out), _ptr(scratch), nbytes, _stream(),
          launches=2 if scratch is not None and V > 4 * 2048 else 1)


def sample(logits: torch.Tensor, temperature: float, state_index: torch.Tensor,
           states: torch.Tensor, out: torch.Tensor) -> None:
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert states.dtype == torch.int64 and state_index.dtype == torch.int32
    _call("sampling", "mb_sample", [_vp, _ll, _i, _i, _d, _vp, _vp, _vp, _vp],
          _ptr(logits), logits.stride(0), rows, V, float(temperature), _ptr(state_index),
          _ptr(states), _ptr(out), _stream())


# ------------------------------------------------------------------------------ tensor cores
def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    lib = build.load_library("gemm_tc")
    f = lib.mb_gemm_tc_supported
    if f.argtypes is None:
        f.argtypes = [_vp, _i, _vp, _i, _i, _i]
        f.restype = _i
    return bool(f(_ptr(a), a.stride(0), _ptr(w), a.shape[0], w.shape[0], w.shape[1]))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, add: bool,
            workspace: Optional[torch.Tensor], error: torch.Tensor, sms: int,
            swiglu: bool = False, defer: bool = False, act: Optional[int] = None) -> int:
    """c = a · wᵀ (or c += for a float32 c) with bfloat16 a [M, K] and w [N, K] on the tensor
    cores; ``swiglu``: w's rows alternate gate and up and c [M, N / 2] = silu(gate) · up.
    ``act`` (ACT_SILU, ACT_GELU_TANH, ACT_RELU_SQUARED): c = act(a · wᵀ), in the epilogue.
    ``workspace``: float32 scratch for split sums; ``error``: int32 device word. ``defer``:
    when K was split (the return value, the number of splits, is above 1) the partial sums stay
    in the workspace as [splits, M, N] and c is not touched."""
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert a.stride(1) == 1 and c.stride(1) == 1 and c.shape == (M, N // 2 if swiglu else N)
    _contig(w, "the weight")
    epilogue = 3 if swiglu else (1 if add else 0)
    if act is not None:
        assert epilogue == 0 and act in (ACT_SILU, ACT_GELU_TANH, ACT_RELU_SQUARED)
        epilogue |= (act + 1) << 8
    _call("gemm_tc", "mb_gemm_tc",
          [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _ll, _i, _vp, _i, _vp],
          _ptr(a), a.stride(0), _ptr(w), _ptr(c), code_of(c.dtype), c.stride(0), M, N, K,
          epilogue, _ptr(workspace),
          workspace.numel() if workspace is not None else 0, 1 if defer else 0,
          _ptr(error), sms, _stream())
    # the split of K adds one kernel that sums the partial products
    lib = build.load_library("gemm_tc")
    Launches.count += lib.mb_gemm_tc_last_launches() - 1
    return lib.mb_gemm_tc_last_splits()


def gemm_tc_gated(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, act: int,
                  pair_bias: Optional[torch.Tensor], error: torch.Tensor, sms: int) -> None:
    """c [M, N / 2] = act(gate + bias) * (up + bias) for a bfloat16 weight [N, K] whose rows
    alternate gate and up (``pair_bias`` [N] bfloat16 alternates likewise, or None), in the
    epilogue of the tensor-core product."""
    M, Kd = a.shape
    N = w.shape[0]
    assert a.dtype == w.dtype == c.dtype == torch.bfloat16 and w.shape[1] == Kd
    assert a.stride(1) == 1 and c.stride(1) == 1 and c.shape == (M, N // 2)
    _contig(w, "the weight")
    if pair_bias is not None:
        assert pair_bias.dtype == torch.bfloat16 and pair_bias.numel() == N
    _call("gemm_tc", "mb_gemm_tc_gated", [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp],
          _ptr(a), a.stride(0), _ptr(w), _ptr(c), c.stride(0), M, N, Kd, act, _ptr(pair_bias),
          _ptr(error), sms, _stream())


def wait_selftest(error: torch.Tensor, code: int, tries: int = 2048) -> bool:
    """Runs one bounded wait that nothing ends (a barrier without anyone to arrive at it),
    with a limit of ``tries`` polls. True if the wait gave up, as it must; ``error`` (int32
    device word) then holds ``code``. The kernel returns by itself either way."""
    gave_up = torch.zeros(1, dtype=torch.int32, device=error.device)
    _call("gemm_tc", "mb_wait_selftest", [_vp, _i, _c.c_uint, _vp, _vp],
          _ptr(error), code, tries, _ptr(gave_up), _stream())
    return bool(gave_up.item())


def advance_decode(tok_ids: torch.Tensor, tok_pos: torch.Tensor, chosen: torch.Tensor,
                   history: Optional[torch.Tensor],
                   seq_past: Optional[torch.Tensor] = None) -> None:
    """The chosen tokens become the next step's ids, every position moves on by one;
    ``seq_past`` (what every sequence held before the step) moves on with them."""
    B = tok_ids.numel()
    assert chosen.dtype == torch.int32 and chosen.numel() == B
    assert seq_past is None or (seq_past.dtype == torch.int32 and seq_past.numel() == B)
    _call("elementwise", "mb_advance_decode", [_vp, _vp, _vp, _vp, _vp, _i, _vp],
          _ptr(tok_ids), _ptr(tok_pos), _ptr(chosen), _ptr(history), _ptr(seq_past), B,
          _stream())


def sample_filtered(logits: torch.Tensor, sampling, state_index: torch.Tensor,
                    states: torch.Tensor, scratch: torch.Tensor, out: torch.Tensor) -> None:
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert scratch.dtype == torch.int64 and scratch.is_contiguous() and scratch.shape[0] >= rows
    _call("sampling", "mb_sample_filtered",
          [_vp, _ll, _i, _i, _d, _i, _d, _d, _vp, _vp, _vp, _ll, _vp, _vp],
          _ptr(logits), logits.stride(0), rows, V, float(sampling.temperature),
          int(sampling.top_k), float(sampling.top_p), float(sampling.min_p), _ptr(state_index),
          _ptr(states), _ptr(scratch), scratch.shape[1], _ptr(out), _stream())


def attention_decode(q: torch.Tensor, q_stride: int, out: torch.Tensor, step, line, nh, nkv, hd,
                     window: int, scale: float, splits: int, scratch: torch.Tensor,
                     error: Optional[torch.Tensor] = None,
                     sink: Optional[torch.Tensor] = None, softcap: float = 0.0,
                     gate: Optional[torch.Tensor] = None, gate_stride: int = 0,
                     slopes: Optional[torch.Tensor] = None, keep_first: int = 0) -> None:
    """Attention of single tokens (a decode step) over the paged cache on the tensor cores; the
    pages of a sequence are dealt out over ``splits`` CTAs. ``softcap``, ``gate``, ``slopes``
    and ``keep_first`` as for ``attention_simt``."""
    T = out.shape[0]
    _contig(out, "out")
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert scratch.dtype == torch.float32 and scratch.is_contiguous()
    assert gate is None or gate.dtype == torch.bfloat16
    _call("attention_mma", "mb_attention_decode",
          [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _f, _i,
           _vp, _ll, _vp, _vp, _f, _vp, _i, _vp, _i, _vp],
          _ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(line.k), _ptr(line.v),
          _ptr(line.page_table), line.max_pages, line.ring_pages, _ptr(step.tok_slot),
          _ptr(step.tok_pos), T, nh, nkv, hd, window, float(scale),
          splits, _ptr(scratch), scratch.numel(), _ptr(error), _ptr(sink), float(softcap),
          _ptr(gate), gate_stride, _ptr(slopes), int(keep_first), _stream(), launches=2)


def attention_decode_clusters(q: torch.Tensor, q_stride: int, out: torch.Tensor, step, line, nh,
                              nkv, hd, window: int, scale: float, splits: int,
                              error: Optional[torch.Tensor] = None,
                              sink: Optional[torch.Tensor] = None, softcap: float = 0.0,
                              gate: Optional[torch.Tensor] = None, gate_stride: int = 0,
                              slopes: Optional[torch.Tensor] = None,
                              keep_first: int = 0) -> None:
    """``attention_decode`` with the splits of a (token, group of heads) as one thread-block
    cluster that merges through its shared memory: no scratch, one kernel; at most 8 splits."""
    T = out.shape[0]
    _contig(out, "out")
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert gate is None or gate.dtype == torch.bfloat16
    _call("attention_mma", "mb_attention_decode_clusters",
          [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _f, _i,
           _vp, _vp, _f, _vp, _i, _vp, _i, _vp],
          _ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(line.k), _ptr(line.v),
          _ptr(line.page_table), line.max_pages, line.ring_pages, _ptr(step.tok_slot),
          _ptr(step.tok_pos), T, nh, nkv, hd, window, float(scale), splits, _ptr(error),
          _ptr(sink), float(softcap), _ptr(gate), gate_stride, _ptr(slopes), int(keep_first),
          _stream())


def attention_prefill(q: torch.Tensor, q_stride: int, out: torch.Tensor, step, line, nh, nkv,
                      hd, window: int, scale: float,
                      error: Optional[torch.Tensor] = None,
                      sink: Optional[torch.Tensor] = None, softcap: float = 0.0,
                      gate: Optional[torch.Tensor] = None, gate_stride: int = 0,
                      slopes: Optional[torch.Tensor] = None, keep_first: int = 0) -> None:
    """Causal attention of every sequence's new tokens over the paged cache on the tensor
    cores (the cache already holds their keys and values)."""
    _contig(out, "out")
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert gate is None or gate.dtype == torch.bfloat16
    _call("attention_mma", "mb_attention_prefill",
          [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f,
           _vp, _vp, _f, _vp, _i, _vp, _i, _vp],
          _ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(line.k), _ptr(line.v),
          _ptr(line.page_table), line.max_pages, line.ring_pages, _ptr(step.seq_start),
          _ptr(step.seq_past), _ptr(step.seq_slot), step.B, step.max_new, nh, nkv, hd, window,
          float(scale), _ptr(error), _ptr(sink), float(softcap), _ptr(gate), gate_stride,
          _ptr(slopes), int(keep_first), _stream())


def attention_prefill_tc(q: torch.Tensor, q_stride: int, out: torch.Tensor, step, line, nh, nkv,
                         hd, window: int, scale: float, error: torch.Tensor,
                         sink: Optional[torch.Tensor] = None, softcap: float = 0.0,
                         gate: Optional[torch.Tensor] = None, gate_stride: int = 0) -> None:
    """The prefill attention on tcgen05 (heads of 128 values): S and O in tensor memory, Q, K
    and V tiles by TMA."""
    _contig(out, "out")
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and q.stride(1) == 1
    assert gate is None or gate.dtype == torch.bfloat16
    pool_rows = line.k.shape[0] * line.k.shape[1] * line.k.shape[2]
    _call("attention_tc", "mb_attention_prefill_tc",
          [_vp, _i, _i, _vp, _i, _vp, _vp, _ll, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i,
           _i, _i, _f, _vp, _vp, _f, _vp, _i, _vp],
          _ptr(q), q_stride, nh * hd, _ptr(out), out.stride(0), _ptr(line.k), _ptr(line.v),
          pool_rows, _ptr(line.page_table), line.max_pages, line.ring_pages,
          _ptr(step.seq_start), _ptr(step.seq_past), _ptr(step.seq_slot), step.B, q.shape[0],
          step.max_new, nh, nkv, hd, window, float(scale), _ptr(error), _ptr(sink),
          float(softcap), _ptr(gate), gate_stride, _stream())
