"""Python entry to the hand-written sm_100a kernels.

Each function checks shapes, types and contiguity, refuses what its kernel does
not take with a clear error, and launches on torch's current CUDA stream through
the library's C entry point.  Nothing here computes on the CPU and nothing falls
back to a library routine: a missing or failing extension raises.

The reference has the same layer: safe wrappers that check sizes before they hand
raw pointers to ``extern "C"`` launchers (crates/airun-cuda/src/ops.rs:1-6, :290-330;
the launchers at crates/airun-cuda/kernels/ops.cu:2222-2578).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_float, c_void_p
from typing import Optional

import torch

from ..csrc import build

DT_F32, DT_BF16 = 0, 1
ROPE_NONE, ROPE_NEOX, ROPE_INTERLEAVED = 0, 1, 2
_DT = {torch.float32: DT_F32, torch.bfloat16: DT_BF16}

DEV_ERR_BITS = {1: "a block-table entry outside the page pool", 2: "a token naming a request outside the batch",
                4: "a token id outside the vocabulary", 8: "a bounded device-side wait ran out"}


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        raise KernelError(f"dtype {t.dtype} is not handled by the kernels (float32 and bfloat16 are)")
    return _DT[t.dtype]


def _p(t: Optional[torch.Tensor]):
    return None if t is None else c_void_p(t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None:
            _need(t.is_cuda, "kernel arguments must live on the GPU (there is no CPU path)")


LAUNCHES = [0]          # kernels launched through this module (CUDA-graph replays are counted by their owner)


def _check(status: int, what: str) -> None:
    if status == 0:
        LAUNCHES[0] += 1
        return
    if status == 1000:
        raise KernelError(f"{what}: the kernel refuses these sizes or pointers")
    if status == 1001:
        raise KernelError(f"{what}: this combination of types is not supported")
    raise KernelError(f"{what}: CUDA error {status} at launch")


_SIGS = {}


def _fn(lib_name: str, fn_name: str, argtypes, defines=None):
    key = (lib_name, fn_name, tuple(sorted((defines or {}).items())))
    f = _SIGS.get(key)
    if f is None:
        lib = build.load(lib_name, defines)
        f = getattr(lib, fn_name)
        f.argtypes = argtypes
        f.restype = c_int
        _SIGS[key] = f
    return f


def required_libraries(dtype: torch.dtype, head_dim: int):
    """(name, defines) of every library a model of this dtype and head size uses."""
    libs = [("elementwise", None), ("gemm_simt", None), ("qkv_post", None),
            ("attention_generic", None), ("sampling", None), ("linear_attention", None), ("diff_attention", None),
            ("recurrent_state", None), ("latent_attention", None), ("moe", None), ("sigmoid_attention", None),
            ("streams", None), ("softmax_attention", None)]
    return libs


# ---------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None,
          scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] widened to float32 (times ``scale``; 1 leaves the values as they are)."""
    _cuda(table, ids, out, err)
    _need(table.dim() == 2 and table.is_contiguous(), "embedding table must be a contiguous [V, H] tensor")
    _need(ids.dtype == torch.int32 and ids.dim() == 1 and ids.is_contiguous(), "ids must be int32 [T]")
    T, (V, H) = ids.shape[0], table.shape
    _need(out.dtype == torch.float32 and tuple(out.shape) == (T, H) and out.is_contiguous(),
          "embedding output must be float32 [T, H]")
    f = _fn("elementwise", "airun_embed",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(f(_p(table), _dt(table), _p(ids), _p(out), T, H, V, float(scale), _p(err), _stream()), "embed")


def soft_cap(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap), in place."""
    _cuda(x)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "soft_cap takes a contiguous float32 tensor")
    _need(cap > 0.0, "the cap must be positive")
    f = _fn("elementwise", "airun_soft_cap", [c_void_p, c_longlong, c_float, c_void_p])
    _check(f(_p(x), x.numel(), float(cap), _stream()), "soft_cap")


def copy_pages(pool: torch.Tensor, pairs: torch.Tensor, err: Optional[torch.Tensor] = None) -> None:
    """pool: [owners, pages, ...] cache pages of one group; pairs: int32 [n, 2] (source page, destination page) on
    the device.  Every owner layer's page ``dst`` becomes a copy of its page ``src``."""
    _cuda(pool, pairs, err)
    _need(pool.dim() >= 3 and pool.is_contiguous(), "pool must be contiguous [owners, pages, ...]")
    _need(pairs.dtype == torch.int32 and pairs.dim() == 2 and pairs.shape[1] == 2 and pairs.is_contiguous(),
          "pairs must be int32 [n, 2]")
    page_bytes = pool[0, 0].numel() * pool.element_size()
    _need(page_bytes % 16 == 0, "a page must be a multiple of 16 bytes")
    f = _fn("elementwise", "airun_copy_pages", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_p(pool), pool.shape[0], pool.shape[1], page_bytes, _p(pairs), pairs.shape[0], _p(err), _stream()), "copy_pages")


def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, out: torch.Tensor,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """out = rmsnorm(x [+ delta]) * weight.

    With ``delta`` and no ``rows`` the sum is written back into ``x`` (the
    residual stream).  With ``rows`` only those rows are normed, into
    out[0..len(rows)), and ``x`` is left as it is.
    """
    _cuda(x, weight, out, delta, rows)
    _need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "x must be float32 [T, n]")
    n = x.shape[1]
    if weight is not None:
        _need(weight.dtype == torch.float32 and tuple(weight.shape) == (n,) and weight.is_contiguous(),
              "norm weight must be float32 [n]")
    if delta is not None:
        _need(delta.dtype == torch.float32 and delta.shape == x.shape and delta.is_contiguous(),
              "delta must match x")
    n_rows = x.shape[0]
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), "rows must be int32 [R]")
        n_rows = rows.shape[0]
    _need(out.dim() == 2 and out.shape[0] >= n_rows and out.shape[1] == n and out.is_contiguous(),
          "norm output must be [rows, n]")
    f = _fn("elementwise", "airun_rmsnorm",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    write_back = 1 if (delta is not None and rows is None) else 0
    _check(f(_p(x), _p(delta), _p(weight), _p(out), _dt(out), _p(rows), n_rows, n, float(eps), write_back,
             _stream()), "rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, group: int) -> None:
    """out[t, i] = silu(g) * u where gate and up columns alternate in blocks of ``group``."""
    _cuda(gate_up, out)
    _need(gate_up.dim() == 2 and out.dim() == 2 and gate_up.is_contiguous() and out.is_contiguous(),
          "swiglu takes contiguous [T, 2I] and [T, I]")
    T, I = out.shape
    _need(gate_up.shape[0] == T and gate_up.shape[1] == 2 * I, "swiglu input must be [T, 2I]")
    f = _fn("elementwise", "airun_swiglu", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_p(gate_up), _dt(gate_up), _p(out), _dt(out), T, I, int(group), _stream()), "swiglu")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(src, rows, out)
    _need(src.dim() == 2 and src.is_contiguous() and out.is_contiguous() and out.dtype == src.dtype,
          "gather_rows takes contiguous 2-d tensors of one type")
    _need(rows.dtype == torch.int32 and rows.is_contiguous(), "rows must be int32")
    rb = src.shape[1] * src.element_size()
    _need(rb % 4 == 0, "row size must be a multiple of 4 bytes")
    _need(out.shape[0] >= rows.shape[0] and out.shape[1] == src.shape[1], "gather output too small")
    f = _fn("elementwise", "airun_gather_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(src), _p(out), _p(rows), rows.shape[0], rb, _stream()), "gather_rows")


def dyt_norm(x: torch.Tensor, alpha: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, out: torch.Tensor,
             delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
             add_vec: Optional[torch.Tensor] = None) -> None:
    """out = tanh(alpha * v) * weight + bias with v = x [+ delta] [+ add_vec] (``add_vec``: one row [n] added
    to every token).  With ``delta`` or ``add_vec`` and no ``rows`` the sum is written back into ``x``; with
    ``rows`` only those rows are normed, into out[0..len(rows)), and ``x`` is left as it is."""
    _cuda(x, alpha, weight, bias, out, delta, rows, add_vec)
    _need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "x must be float32 [T, n]")
    n = x.shape[1]
    for w in (weight, bias):
        _need(w.dtype == torch.float32 and tuple(w.shape) == (n,) and w.is_contiguous(), "norm weight and bias must be float32 [n]")
    _need(alpha.dtype == torch.float32 and alpha.numel() == 1, "alpha must be one float32 number")
    if delta is not None:
        _need(delta.dtype == torch.float32 and delta.shape == x.shape and delta.is_contiguous(), "delta must match x")
    if add_vec is not None:
        _need(add_vec.dtype == torch.float32 and tuple(add_vec.shape) == (n,) and add_vec.is_contiguous(),
              "add_vec must be float32 [n]")
    n_rows = x.shape[0]
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), "rows must be int32 [R]")
        n_rows = rows.shape[0]
    _need(out.dim() == 2 and out.shape[0] >= n_rows and out.shape[1] == n and out.is_contiguous(),
          "norm output must be [rows, n]")
    f = _fn("elementwise", "airun_dyt_norm",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
             c_void_p])
    write_back = 1 if ((delta is not None or add_vec is not None) and rows is None) else 0
    _check(f(_p(x), _p(delta), _p(add_vec), _p(alpha), _p(weight), _p(bias), _p(out), _dt(out), _p(rows), n_rows, n,
             write_back, _stream()), "dyt_norm")


def add_rows(x: torch.Tensor, delta: Optional[torch.Tensor] = None, vec: Optional[torch.Tensor] = None) -> None:
    """x += delta (same shape) and/or x[t] += vec for every row t, in place, float32."""
    _cuda(x, delta, vec)
    _need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "x must be contiguous float32 [T, n]")
    if delta is not None:
        _need(delta.dtype == torch.float32 and delta.shape == x.shape and delta.is_contiguous(), "delta must match x")
    if vec is not None:
        _need(vec.dtype == torch.float32 and tuple(vec.shape) == (x.shape[1],) and vec.is_contiguous(), "vec must be float32 [n]")
    f = _fn("elementwise", "airun_add_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(x), _p(delta), _p(vec), x.shape[0], x.shape[1], _stream()), "add_rows")


def glu_clamped(gate_up: torch.Tensor, out: torch.Tensor, group: int, limit: float, slope: float) -> None:
    """out[t, i] = g * sigmoid(slope * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit); gate and
    up columns alternate in blocks of ``group``.  ``out`` may be a column slice of a wider buffer."""
    _cuda(gate_up, out)
    _need(gate_up.dim() == 2 and out.dim() == 2 and gate_up.is_contiguous() and out.stride(1) == 1
          and gate_up.dtype == torch.float32, "glu_clamped takes contiguous float32 [T, 2I] and row-major [T, I]")
    T, I = out.shape
    _need(gate_up.shape[0] == T and gate_up.shape[1] == 2 * I, "glu_clamped input must be [T, 2I]")
    f = _fn("elementwise", "airun_glu_clamped",
            [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_float, c_float, c_void_p])
    _check(f(_p(gate_up), _dt(gate_up), _p(out), _dt(out), T, I, int(group), out.stride(0) if T > 1 else max(I, out.stride(0)),
             float(limit), float(slope), _stream()), "glu_clamped")


def postnorm_add(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, mult: float,
                 cast: Optional[torch.Tensor] = None) -> None:
    """x += mult * y / rms(y) * weight row by row (the norm sits on the sub-layer's output); with ``cast`` the new x
    is also written there in its type, as the input of the sub-layer that follows."""
    _cuda(x, y, weight, cast)
    _need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "x must be contiguous float32 [T, n]")
    T, n = x.shape
    _need(y.dtype == torch.float32 and y.shape == x.shape and y.is_contiguous(), "y must match x")
    _need(weight.dtype == torch.float32 and tuple(weight.shape) == (n,) and weight.is_contiguous(), "norm weight must be float32 [n]")
    if cast is not None:
        _need(tuple(cast.shape) == (T, n) and cast.is_contiguous(), "cast must be contiguous [T, n]")
    f = _fn("elementwise", "airun_postnorm_add",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p])
    _check(f(_p(x), _p(y), _p(weight), _p(cast), _dt(cast) if cast is not None else DT_F32, T, n, float(eps), float(mult),
             _stream()), "postnorm_add")


def cast_f32(src: torch.Tensor, out: torch.Tensor) -> None:
    """out = src (float32) in out's type."""
    _cuda(src, out)
    _need(src.dtype == torch.float32 and src.is_contiguous() and out.is_contiguous() and out.numel() == src.numel(),
          "cast_f32 takes contiguous tensors of one size")
    f = _fn("elementwise", "airun_cast_f32", [c_void_p, c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_p(src), _p(out), _dt(out), src.numel(), _stream()), "cast_f32")


def rmsnorm_pair(x: torch.Tensor, w1: torch.Tensor, out1: torch.Tensor, w2: torch.Tensor, out2: torch.Tensor, eps: float,
                 delta: Optional[torch.Tensor] = None) -> None:
    """out1 = rmsnorm(x [+ delta]) * w1 and out2 = the same row * w2, in one pass; with ``delta`` the sum becomes x."""
    _cuda(x, w1, out1, w2, out2, delta)
    _need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "x must be float32 [T, n]")
    T, n = x.shape
    for w in (w1, w2):
        _need(w.dtype == torch.float32 and tuple(w.shape) == (n,) and w.is_contiguous(), "norm weights must be float32 [n]")
    for o in (out1, out2):
        _need(tuple(o.shape) == (T, n) and o.is_contiguous() and o.dtype == out1.dtype, "norm outputs must be [T, n] of one type")
    if delta is not None:
        _need(delta.dtype == torch.float32 and delta.shape == x.shape and delta.is_contiguous(), "delta must match x")
    f = _fn("elementwise", "airun_rmsnorm_pair",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_p(x), _p(delta), _p(w1), _p(out1), _p(w2), _p(out2), _dt(out1), None, T, n, float(eps),
             1 if delta is not None else 0, _stream()), "rmsnorm_pair")


ACT_RELU2, ACT_SILU, ACT_GELU_TANH, ACT_RELU, ACT_GELU_ERF = 0, 1, 2, 3, 4
ACTIVATIONS = {"relu2": ACT_RELU2, "silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH, "relu": ACT_RELU, "gelu_erf": ACT_GELU_ERF}


def act(src: torch.Tensor, out: torch.Tensor, mode: int) -> None:
    """out = f(src) element by element: relu(z)^2, z sigmoid(z), the tanh or the erf form of GELU or relu(z) (``ACT_*``); src
    float32 [T, n], out [T, n] in its own type (a column slice of a wider buffer is fine)."""
    _cuda(src, out)
    _need(src.dtype == torch.float32 and src.dim() == 2 and src.is_contiguous(), "src must be contiguous float32 [T, n]")
    T, n = src.shape
    _need(tuple(out.shape) == (T, n) and out.stride(1) == 1, "out must be row-major [T, n]")
    f = _fn("elementwise", "airun_act", [c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_int, c_void_p])
    _check(f(_p(src), _p(out), _dt(out), T, n, _row_stride(out), int(mode), _stream()), "act")


def gated_sum(out: torch.Tensor, y1: torch.Tensor, g1: Optional[torch.Tensor] = None, c1: Optional[torch.Tensor] = None,
              s1: Optional[torch.Tensor] = None, y2: Optional[torch.Tensor] = None, g2: Optional[torch.Tensor] = None,
              c2: Optional[torch.Tensor] = None, s2: Optional[torch.Tensor] = None) -> None:
    """out = s1 * sigmoid(g1 + c1) * y1 [+ s2 * sigmoid(g2 + c2) * y2]: y float32 [T, n], g float32 [T, n] (column slices
    are fine), c and s float32 [n]; a missing g means no gate, a missing s no scale.  ``out`` may be y1."""
    _cuda(out, y1, g1, c1, s1, y2, g2, c2, s2)
    _need(y1.dtype == torch.float32 and y1.dim() == 2 and y1.is_contiguous(), "y1 must be contiguous float32 [T, n]")
    T, n = y1.shape
    _need(out.dtype == torch.float32 and out.shape == y1.shape and out.is_contiguous(), "out must match y1")
    if y2 is not None:
        _need(y2.dtype == torch.float32 and y2.shape == y1.shape and y2.is_contiguous(), "y2 must match y1")
    for g in (g1, g2):
        if g is not None:
            _rows_f32(g, "a gate")
            _need(tuple(g.shape) == (T, n), "a gate must be [T, n]")
    for v in (c1, s1, c2, s2):
        if v is not None:
            _need(v.dtype == torch.float32 and tuple(v.shape) == (n,) and v.is_contiguous(), "biases and scales must be float32 [n]")
    f = _fn("elementwise", "airun_gated_sum",
            [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_void_p])
    _check(f(_p(y1), _p(g1), _row_stride(g1) if g1 is not None else 0, _p(c1), _p(s1), _p(y2), _p(g2),
             _row_stride(g2) if g2 is not None else 0, _p(c2), _p(s2), _p(out), T, n, _stream()), "gated_sum")


def scale_(x: torch.Tensor, factor: float) -> None:
    """x *= factor, in place."""
    _cuda(x)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "scale_ takes a contiguous float32 tensor")
    f = _fn("elementwise", "airun_scale", [c_void_p, c_longlong, c_float, c_void_p])
    _check(f(_p(x), x.numel(), float(factor), _stream()), "scale")


# ---------------------------------------------------------------- gated linear attention
def _rows_f32(t: torch.Tensor, what: str) -> None:
    _need(t.dtype == torch.float32 and t.dim() == 2 and t.stride(1) == 1, f"{what} must be float32 rows (a column slice is fine)")


def _row_stride(t: torch.Tensor) -> int:
    return t.stride(0) if t.shape[0] > 1 else max(t.shape[1], t.stride(0))


def gla_decay(low: torch.Tensor, w2: torch.Tensor, bias: Optional[torch.Tensor], tau: float, out: torch.Tensor,
                  req_of_token: torch.Tensor) -> None:
    """out[t, c] = exp(logsigmoid(bias[c] + low[t] . w2[c]) / tau): the decay sigmoid(z)^(1/tau), in (0, 1)."""
    _cuda(low, w2, bias, out, req_of_token)
    _rows_f32(low, "low")
    T, rank = low.shape
    n = w2.shape[0]
    _need(w2.dim() == 2 and w2.shape[1] == rank and w2.is_contiguous(), "w2 must be contiguous [n, rank]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and tuple(bias.shape) == (n,) and bias.is_contiguous(), "bias must be float32 [n]")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (T, n) and out.is_contiguous(), "out must be float32 [T, n]")
    _need(req_of_token.dtype == torch.int32 and req_of_token.shape[0] >= T, "req_of_token must be int32 [T]")
    f = _fn("linear_attention", "airun_gla_decay",
            [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(f(_p(low), _row_stride(low), _p(w2), _dt(w2), _p(bias), _p(out), T, n, rank, float(tau), _p(req_of_token),
             _stream()), "gla_decay")


def gla_recurrent(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
                  cu_tokens: torch.Tensor, state_slots: torch.Tensor, num_reqs: int, out: torch.Tensor,
                  heads: int, D: int, Dv: int, q_scale: float, err: torch.Tensor) -> None:
    """The recurrence S <- diag(a) S + k v^T, o = S^T q * q_scale for the tokens of every request in order.
    ``q``, ``k`` [T, heads*D] and ``v`` [T, heads*Dv] are float32 column slices of ONE buffer (equal row strides);
    ``state`` is [slots, heads, D, Dv] float32 and is updated in place; ``out`` float32 [T, heads*Dv]."""
    _cuda(q, k, v, decay, state, cu_tokens, state_slots, out, err)
    for t, w, name in ((q, heads * D, "q"), (k, heads * D, "k"), (v, heads * Dv, "v")):
        _rows_f32(t, name)
        _need(t.shape[1] == w, f"{name} must have {w} columns")
    T = q.shape[0]
    _need(_row_stride(q) == _row_stride(k) or T <= 1, "q, k and v must share a row stride")
    _need(k.stride(0) == v.stride(0) or T <= 1, "q, k and v must share a row stride")
    _need(decay.dtype == torch.float32 and tuple(decay.shape) == (T, heads * D) and decay.is_contiguous(),
          "decay must be float32 [T, heads*D]")
    _need(state.dtype == torch.float32 and state.dim() == 4 and tuple(state.shape[1:]) == (heads, D, Dv)
          and state[0].is_contiguous(), "state must be float32 [slots, heads, D, Dv]")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (T, heads * Dv) and out.is_contiguous(), "out must be float32 [T, heads*Dv]")
    _need(cu_tokens.dtype == torch.int32 and cu_tokens.numel() >= num_reqs + 1 and state_slots.dtype == torch.int32
          and state_slots.numel() >= num_reqs, "cu_tokens / state_slots must be int32 [R + 1] / [R]")
    _need(D <= 256, f"{D} key channels a head are above the kernel's limit of 256")
    stride = q.stride(0) if T > 1 else max(q.stride(0), k.stride(0), v.stride(0))
    f = _fn("linear_attention", "airun_gla_recurrent",
            [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int,
             c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(f(_p(q), _p(k), _p(v), stride, _p(decay), _p(state), state.stride(0), state.shape[0], _p(cu_tokens),
             _p(state_slots), int(num_reqs), _p(out), heads, D, Dv, float(q_scale), _p(err), _stream()), "gla_recurrent")


def decay_recurrent(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, head_decay: torch.Tensor, in_silu: bool,
                    state: torch.Tensor, cu_tokens: torch.Tensor, state_slots: torch.Tensor, num_reqs: int, out: torch.Tensor,
                    heads: int, D: int, Dv: int, q_scale: float, err: torch.Tensor) -> None:
    """The recurrence with one decay per head, S <- d_h S + k v^T, o = S^T q * q_scale, for the tokens of every request in
    order.  ``q``, ``k`` [T, heads*D] and ``v`` [T, heads*Dv] are float32 column slices of ONE buffer; with ``in_silu``
    they arrive without their activation z sigmoid(z), which the kernel applies.  ``head_decay`` float32 [heads];
    ``state`` [slots, heads, D, Dv] float32, updated in place; ``out`` float32 [T, heads*Dv]."""
    _cuda(q, k, v, head_decay, state, cu_tokens, state_slots, out, err)
    for t, w, name in ((q, heads * D, "q"), (k, heads * D, "k"), (v, heads * Dv, "v")):
        _rows_f32(t, name)
        _need(t.shape[1] == w, f"{name} must have {w} columns")
    T = q.shape[0]
    _need((q.stride(0) == k.stride(0) == v.stride(0)) or T <= 1, "q, k and v must share a row stride")
    _need(head_decay.dtype == torch.float32 and head_decay.numel() == heads and head_decay.is_contiguous(),
          "head_decay must be float32 [heads]")
    _need(state.dtype == torch.float32 and state.dim() == 4 and tuple(state.shape[1:]) == (heads, D, Dv)
          and state[0].is_contiguous(), "state must be float32 [slots, heads, D, Dv]")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (T, heads * Dv) and out.is_contiguous(), "out must be float32 [T, heads*Dv]")
    _need(cu_tokens.dtype == torch.int32 and cu_tokens.numel() >= num_reqs + 1 and state_slots.dtype == torch.int32
          and state_slots.numel() >= num_reqs, "cu_tokens / state_slots must be int32 [R + 1] / [R]")
    _need(D <= 256, f"{D} key channels a head are above the kernel's limit of 256")
    stride = q.stride(0) if T > 1 else max(q.stride(0), k.stride(0), v.stride(0))
    f = _fn("linear_attention", "airun_decay_recurrent",
            [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int,
             c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(f(_p(q), _p(k), _p(v), stride, _p(head_decay), 1 if in_silu else 0, _p(state), state.stride(0), state.shape[0],
             _p(cu_tokens), _p(state_slots), int(num_reqs), _p(out), heads, D, Dv, float(q_scale), _p(err), _stream()),
           "decay_recurrent")


def rownorm_gate(o: torch.Tensor, gate: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float, out: torch.Tensor,
                 req_of_token: torch.Tensor, scale: float = 1.0) -> None:
    """out = scale * o / rms(o) * weight * sigmoid(gate), the root mean square over a token's WHOLE row (all heads at
    once).  ``o`` float32 [T, n] contiguous, ``gate`` float32 rows (a column slice is fine), ``out`` [T, n] rows."""
    _cuda(o, gate, weight, out, req_of_token)
    T, n = o.shape
    _need(o.dtype == torch.float32 and o.is_contiguous(), "o must be contiguous float32 [T, n]")
    if gate is not None:
        _rows_f32(gate, "gate")
        _need(tuple(gate.shape) == (T, n), "gate must be [T, n]")
    if weight is not None:
        _need(weight.dtype == torch.float32 and weight.numel() == n and weight.is_contiguous(), "the norm weight must be float32 [n]")
    _need(tuple(out.shape) == (T, n) and out.stride(1) == 1, "out must be row-major [T, n]")
    f = _fn("linear_attention", "airun_rownorm_gate",
            [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_float, c_float, c_void_p, c_void_p])
    _check(f(_p(o), _p(gate), _row_stride(gate) if gate is not None else n, _p(weight), _p(out), _dt(out), _row_stride(out), T, n,
             float(eps), float(scale), _p(req_of_token), _stream()), "rownorm_gate")


GATE_SILU, GATE_SIGMOID, GATE_AS_IS = 0, 1, 2


def gla_out_gate(o: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor], eps: float, out: torch.Tensor,
                 heads: int, Dv: int, req_of_token: torch.Tensor, gate_act: int = GATE_SILU,
                 weight_per_head: bool = False) -> None:
    """out[t, h] = o[t, h] / rms(o[t, h]) * weight * f(gate[t, h]) per head of ``Dv`` values; f is silu, sigmoid
    or the identity (``gate_act``); ``weight`` is [Dv], shared by the heads, or [heads * Dv] (``weight_per_head``)."""
    _cuda(o, gate, weight, out, req_of_token)
    T = o.shape[0]
    _need(o.dtype == torch.float32 and tuple(o.shape) == (T, heads * Dv) and o.is_contiguous(), "o must be float32 [T, heads*Dv]")
    _rows_f32(gate, "gate")
    _need(tuple(gate.shape) == (T, heads * Dv), "gate must be [T, heads*Dv]")
    _need(out.dim() == 2 and tuple(out.shape) == (T, heads * Dv) and out.stride(1) == 1, "out must be row-major [T, heads*Dv]")
    if weight is not None:
        _need(weight.dtype == torch.float32 and weight.numel() == (heads * Dv if weight_per_head else Dv)
              and weight.is_contiguous(), "weight must be float32 [Dv] (or [heads * Dv] per head)")
    f = _fn("linear_attention", "airun_gla_out_gate",
            [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_float, c_void_p,
             c_int, c_int, c_void_p])
    _check(f(_p(o), _p(gate), _row_stride(gate), _p(weight), _p(out), _dt(out), _row_stride(out), T, heads, Dv, float(eps),
             _p(req_of_token), int(gate_act), 1 if weight_per_head else 0, _stream()), "gla_out_gate")


LOWRANK_POW_SIGMOID, LOWRANK_EXP_SOFTPLUS, LOWRANK_SIGMOID, LOWRANK_EXP_NEG_EXP = 0, 1, 2, 3


def lowrank_act(low: torch.Tensor, w2: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                req_of_token: torch.Tensor, mode: int, in_tanh: bool = False, tau: float = 1.0,
                group_param: Optional[torch.Tensor] = None, group: int = 0) -> None:
    """The second half of a low-rank pair with the function that follows it, in float32:
    z[t, c] = bias[c] + f(low[t]) . w2[c] (f = tanh with ``in_tanh``), out = sigmoid(z)^(1/tau),
    exp(-exp(group_param[c // group]) * softplus(z)), sigmoid(z) or exp(-exp(z)) by ``mode``."""
    _cuda(low, w2, bias, out, req_of_token, group_param)
    _rows_f32(low, "low")
    T, rank = low.shape
    n = w2.shape[0]
    _need(w2.dim() == 2 and w2.shape[1] == rank and w2.is_contiguous(), "w2 must be contiguous [n, rank]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n and bias.is_contiguous(), "bias must be float32 [n]")
    if group_param is not None:
        _need(group_param.dtype == torch.float32 and group > 0 and group_param.numel() * group == n and group_param.is_contiguous(),
              "group_param must be float32 [n / group]")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (T, n) and out.is_contiguous(), "out must be float32 [T, n]")
    _need(req_of_token.dtype == torch.int32 and req_of_token.shape[0] >= T, "req_of_token must be int32 [T]")
    f = _fn("linear_attention", "airun_lowrank_act",
            [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int,
             c_void_p, c_int, c_void_p])
    _check(f(_p(low), _row_stride(low), _p(w2), _dt(w2), _p(bias), _p(out), T, n, rank, float(tau), _p(req_of_token),
             int(mode), 1 if in_tanh else 0, _p(group_param), int(group), _stream()), "lowrank_act")


# ---------------------------------------------------------------- differential attention
def _page_args(pool: torch.Tensor, nkv: int, kd: int, vd: int, page_size: int):
    _need(pool.is_contiguous() and pool.dim() >= 2 and pool[0].numel() == nkv * page_size * (kd + vd),
          f"a cache page must hold {nkv} x {page_size} keys of {kd} and values of {vd}")
    return pool.shape[0]


def qkv_bias_store(proj: torch.Tensor, q_bias, k_bias, v_bias, q_out: torch.Tensor, pool: Optional[torch.Tensor],
                   block_table: Optional[torch.Tensor], positions: torch.Tensor, req_of_token: torch.Tensor,
                   num_reqs: int, page_size: int, q_width: int, nkv: int, kd: int, vd: int, err: torch.Tensor,
                   store: bool = True) -> None:
    """q_out = proj[:, :q_width] + q_bias; the keys (next nkv*kd columns) and values (nkv*vd columns after them) with
    their biases go into the token's cache page (keys of all KV heads, then values)."""
    _cuda(proj, q_bias, k_bias, v_bias, q_out, pool, block_table, positions, req_of_token, err)
    _rows_f32(proj, "proj")
    T = proj.shape[0]
    _need(proj.shape[1] >= q_width + (nkv * (kd + vd) if store else 0), "proj is too narrow for q, k and v")
    _need(tuple(q_out.shape) == (T, q_width) and q_out.is_contiguous(), "q_out must be contiguous [T, q_width]")
    for b, w in ((q_bias, q_width), (k_bias, nkv * kd), (v_bias, nkv * vd)):
        if b is not None:
            _need(b.dtype == torch.float32 and tuple(b.shape) == (w,) and b.is_contiguous(), "a bias must be float32 of its projection's width")
    num_pages = max_blocks = 0
    if store:
        num_pages = _page_args(pool, nkv, kd, vd, page_size)
        _need(pool.dtype == q_out.dtype, "q and the cache pages must share a type")
        _need(block_table is not None and block_table.dtype == torch.int32 and block_table.dim() == 2
              and block_table.stride(1) == 1, "block_table must be int32 [R, max_blocks]")
        max_blocks = block_table.stride(0)
    f = _fn("diff_attention", "airun_qkv_bias_store",
            [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(proj), _row_stride(proj), _p(q_bias), _p(k_bias), _p(v_bias), _p(q_out), _p(pool), _dt(q_out),
             _p(block_table), max_blocks, _p(positions), _p(req_of_token), T, int(num_reqs), num_pages, int(page_size),
             q_width, nkv, kd, vd, 1 if store else 0, _p(err), _stream()), "qkv_bias_store")


def diff_attention(q: torch.Tensor, out: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor,
                   positions: torch.Tensor, req_of_token: torch.Tensor, num_reqs: int, page_size: int,
                   nh: int, nkv: int, D: int, Dv: int, scale: float, cap: float, chunk: int, window: int,
                   lam: float, eps: float, out_scale: float, err: torch.Tensor) -> None:
    """Two attention maps per head over the same values, o = a1 - lam * a2, then o / rms(o) * out_scale per head
    (see csrc/diff_attention.cu); float32 arithmetic, any sizes up to 256."""
    _cuda(q, out, pool, block_table, positions, req_of_token, err)
    T = q.shape[0]
    _need(tuple(q.shape) == (T, nh * 2 * D) and q.is_contiguous(), "q must be contiguous [T, heads*2*D]")
    _need(tuple(out.shape) == (T, nh * Dv) and out.stride(1) == 1 and out.dtype == q.dtype, "out must be row-major [T, heads*Dv] of q's type")
    _need(D <= 256 and Dv <= 256, "head sizes above 256 are not taken")
    _need(nh % nkv == 0, "query heads must be a multiple of KV heads")
    num_pages = _page_args(pool, nkv, 2 * D, Dv, page_size)
    _need(pool.dtype == q.dtype, "q and the cache pages must share a type")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1,
          "block_table must be int32 [R, max_blocks]")
    f = _fn("diff_attention", "airun_diff_attention",
            [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_float, c_float, c_float, c_void_p, c_void_p])
    _check(f(_p(q), _p(out), _row_stride(out), _p(pool), _dt(q), _p(block_table), block_table.stride(0), _p(positions),
             _p(req_of_token), T, int(num_reqs), num_pages, int(page_size), nh, nkv, D, Dv, float(scale), float(cap),
             int(chunk), int(window), float(lam), float(eps), float(out_scale), _p(err), _stream()), "diff_attention")


# ---------------------------------------------------------------- attention without softmax
def qk_rownorm_store(proj: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], eps: float,
                     temp_coef: float, temp_every: int, q_out: torch.Tensor, cache, ctx, q_width: int, nkv: int, kd: int,
                     vd: int, store: bool = True) -> None:
    """q_out = proj[:, :q_width] / rms * q_w * (1 + temp_coef * ln((pos + 1) // temp_every + 1)); the keys (next nkv*kd
    columns, normed over all of them with k_w) and the values (nkv*vd columns after them) go into the token's page.
    The root mean squares run over the whole projection of a token; ``temp_every`` 0: no temperature."""
    pool, block_table = (cache.pool, cache.block_table) if store else (None, None)
    _cuda(proj, q_w, k_w, q_out, pool, block_table)
    _rows_f32(proj, "proj")
    T = proj.shape[0]
    _need(proj.shape[1] >= q_width + (nkv * (kd + vd) if store else 0), "proj is too narrow for q, k and v")
    _need(tuple(q_out.shape) == (T, q_width) and q_out.is_contiguous(), "q_out must be contiguous [T, q_width]")
    for w, n in ((q_w, q_width), (k_w, nkv * kd)):
        if w is not None:
            _need(w.dtype == torch.float32 and tuple(w.shape) == (n,) and w.is_contiguous(), "a norm weight must be float32 of its projection's width")
    num_pages = max_blocks = 0
    if store:
        num_pages = _page_args(pool, nkv, kd, vd, cache.page_size)
        _need(pool.dtype == q_out.dtype, "q and the cache pages must share a type")
        _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1,
              "block_table must be int32 [R, max_blocks]")
        max_blocks = block_table.stride(0)
    f = _fn("sigmoid_attention", "airun_qk_rownorm_store",
            [c_void_p, c_longlong, c_void_p, c_void_p, c_float, c_float, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(proj), _row_stride(proj), _p(q_w), _p(k_w), float(eps), float(temp_coef), int(temp_every), _p(q_out), _p(pool),
             _dt(q_out), _p(block_table), max_blocks, _p(ctx.positions), _p(ctx.req_of_token), T, int(ctx.num_reqs), num_pages,
             int(cache.page_size), q_width, nkv, kd, vd, 1 if store else 0, _p(ctx.err), _stream()), "qk_rownorm_store")


def sigmoid_attention(q: torch.Tensor, out: torch.Tensor, cache, ctx, nh: int, nkv: int, D: int, Dv: int, scale: float,
                      dist_a: Optional[torch.Tensor], dist_b: Optional[torch.Tensor], head_c: Optional[torch.Tensor],
                      window: int = 0) -> None:
    """out[t, h] = sum over the visible keys j of sigmoid(scale * q . k_j - a_h * ln(1 + b_h * (pos - j)) + c_h) * v_j
    (see csrc/sigmoid_attention.cu); float32 arithmetic, any sizes up to 256."""
    pool, block_table = cache.pool, cache.block_table
    _cuda(q, out, pool, block_table, dist_a, dist_b, head_c)
    T = q.shape[0]
    _need(tuple(q.shape) == (T, nh * D) and q.is_contiguous(), "q must be contiguous [T, heads*D]")
    _need(tuple(out.shape) == (T, nh * Dv) and out.stride(1) == 1 and out.dtype == q.dtype, "out must be row-major [T, heads*Dv] of q's type")
    _need(D <= 256 and Dv <= 256, "head sizes above 256 are not taken")
    _need(nh % nkv == 0, "query heads must be a multiple of KV heads")
    num_pages = _page_args(pool, nkv, D, Dv, cache.page_size)
    _need(pool.dtype == q.dtype, "q and the cache pages must share a type")
    for v in (dist_a, dist_b, head_c):
        if v is not None:
            _need(v.dtype == torch.float32 and v.numel() == nh and v.is_contiguous(), "the heads' numbers must be float32 [heads]")
    _need((dist_a is None) == (dist_b is None), "the distance term needs both of its numbers")
    f = _fn("sigmoid_attention", "airun_sigmoid_attention",
            [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_p(q), _p(out), _row_stride(out), _p(pool), _dt(q), _p(block_table), block_table.stride(0), _p(ctx.positions),
             _p(ctx.req_of_token), T, int(ctx.num_reqs), num_pages, int(cache.page_size), nh, nkv, D, Dv, float(scale),
             _p(dist_a), _p(dist_b), _p(head_c), int(window), _p(ctx.err), _stream()), "sigmoid_attention")


# ---------------------------------------------------------------- matrix products
# ---------------------------------------------------------------- a residual of several streams
STREAMS_MAX = 8


def stream_fill(x: torch.Tensor, xs: torch.Tensor) -> None:
    """xs[t, s] = x[t] for every stream s: x float32 [T, H], xs float32 [T, S, H]."""
    _cuda(x, xs)
    T, S, H = xs.shape
    _need(x.dtype == torch.float32 and xs.dtype == torch.float32 and tuple(x.shape) == (T, H) and x.is_contiguous()
          and xs.is_contiguous(), "x / xs must be contiguous float32 [T, H] / [T, S, H]")
    f = _fn("streams", "airun_stream_fill", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(x), _p(xs), T, S, H, _stream()), "stream_fill")


def stream_step(xs: torch.Tensor, y: Optional[torch.Tensor] = None, carry: Optional[torch.Tensor] = None,
                write: Optional[torch.Tensor] = None, mult: float = 1.0, y_bias: Optional[torch.Tensor] = None,
                read: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None, eps: float = 0.0,
                out: Optional[torch.Tensor] = None, req_of_token: Optional[torch.Tensor] = None) -> None:
    """One pass over the streams xs float32 [T, S, H] (csrc/streams.cu).  With ``y`` [T, H] the result of a sub-layer is
    written in: x_t <- sum_s carry[s, t] x_s + mult * write[t] * (y + y_bias), all t from the old streams, in place.
    With ``read`` [S] the next sub-layer's input is formed from the new streams: u = sum_s read[s] x_s, and
    ``out`` = u / rms(u) * norm_w in out's type, or u itself in float32 when there is no ``norm_w``."""
    _cuda(xs, y, carry, write, y_bias, read, norm_w, out, req_of_token)
    _need(xs.dtype == torch.float32 and xs.dim() == 3 and xs.is_contiguous(), "xs must be contiguous float32 [T, S, H]")
    T, S, H = xs.shape
    _need(S <= STREAMS_MAX, f"{S} streams are above the kernel's limit of {STREAMS_MAX}")
    _need(y is not None or read is not None, "nothing to do: neither a result to write nor a read")
    if y is not None:
        _rows_f32(y, "y")
        _need(tuple(y.shape) == (T, H), "y must be [T, H]")
        _need(carry is not None and write is not None and carry.dtype == torch.float32 and write.dtype == torch.float32
              and carry.numel() == S * S and write.numel() == S and carry.is_contiguous() and write.is_contiguous(),
              "carry / write must be float32 [S, S] / [S]")
        if y_bias is not None:
            _need(y_bias.dtype == torch.float32 and y_bias.numel() == H and y_bias.is_contiguous(), "y_bias must be float32 [H]")
    if read is not None:
        _need(read.dtype == torch.float32 and read.numel() == S and read.is_contiguous(), "read must be float32 [S]")
        _need(out is not None and tuple(out.shape) == (T, H) and out.stride(1) == 1, "out must be row-major [T, H]")
        if norm_w is None:
            _need(out.dtype == torch.float32, "without a norm the weighted sum is stored in float32")
        else:
            _need(norm_w.dtype == torch.float32 and norm_w.numel() == H and norm_w.is_contiguous(), "norm_w must be float32 [H]")
    f = _fn("streams", "airun_stream_step",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float,
             c_void_p, c_int, c_longlong, c_void_p, c_void_p])
    _check(f(_p(xs), T, S, H, _p(y), _row_stride(y) if y is not None else H, _p(y_bias), _p(carry), _p(write), float(mult), _p(read),
             _p(norm_w), float(eps), _p(out), _dt(out) if out is not None else DT_F32, _row_stride(out) if out is not None else H,
             _p(req_of_token), _stream()), "stream_step")


# ---------------------------------------------------------------- softmax attention with its options
def qkv_prepare(proj: torch.Tensor, bias: Optional[torch.Tensor], q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                unit_norm: bool, eps: float, rope_kind: int, rotary_dim: int, inv_freq: Optional[torch.Tensor],
                temp_coef: float, temp_every: int, q_out: torch.Tensor, cache, ctx, nh: int, nkv: int, D: int, Dv: int,
                store: bool = True, rope_positions: Optional[torch.Tensor] = None) -> None:
    """What lies between the q/k/v product and the attention (csrc/softmax_attention.cu: qkv_prepare_kernel): biases,
    a weighted root-mean-square norm per head before the rotation (``q_w`` / ``k_w`` float32 [D]), the rotation, an
    unweighted norm per head after it (``unit_norm``), the query temperature; q out, k and v into the token's page.
    ``proj`` float32 rows [q heads | k heads | v heads] (q heads only without ``store``)."""
    _cuda(proj, bias, q_w, k_w, inv_freq, q_out, cache.pool, cache.block_table, ctx.positions, ctx.req_of_token, ctx.err, rope_positions)
    _rows_f32(proj, "proj")
    T = proj.shape[0]
    width = nh * D + (nkv * (D + Dv) if store else 0)
    _need(proj.shape[1] >= width, f"proj must have at least {width} columns")
    _need(q_out.is_contiguous() and tuple(q_out.shape) == (T, nh * D), "q_out must be contiguous [T, heads*D]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() >= width and bias.is_contiguous(), "the biases must be float32 [q | k | v]")
    for w_ in (q_w, k_w):
        _need(w_ is None or (w_.dtype == torch.float32 and w_.numel() == D and w_.is_contiguous()), "a q/k norm weight must be float32 [D]")
    _need(D <= 256, "head sizes above 256 are beyond the kernel")
    pool, bt = cache.pool, cache.block_table
    if store:
        _need(pool.dtype == q_out.dtype and pool.is_contiguous() and pool[0].numel() == nkv * cache.page_size * (D + Dv),
              "the cache pages do not fit the head sizes or the type of q")
    f = _fn("softmax_attention", "airun_qkv_prepare",
            [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_float, c_int,
             c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_void_p, c_void_p])
    _check(f(_p(proj), _row_stride(proj), _p(bias), _p(q_w), _p(k_w), 1 if unit_norm else 0, float(eps), int(rope_kind),
             int(rotary_dim), _p(inv_freq), _p(rope_positions), float(temp_coef), int(temp_every), _p(q_out), _p(pool), _dt(q_out),
             _p(bt), bt.stride(0), _p(ctx.positions), _p(ctx.req_of_token), T, int(ctx.num_reqs), pool.shape[0],
             int(cache.page_size), nh, nkv, D, Dv, 1 if store else 0, _p(ctx.err), _stream()), "qkv_prepare")


def softmax_attention(q: torch.Tensor, out: torch.Tensor, cache, ctx, nh: int, nkv: int, D: int, Dv: int, scale: float,
                      table: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None, window: int = 0,
                      out_scale: float = 1.0) -> None:
    """Softmax attention over cache pages in float32 arithmetic (csrc/softmax_attention.cu: softmax_attention_kernel):
    ``table`` float32 [heads, n] adds table[h, min(i - j, n - 1)] to the scaled score, ``sink`` float32 [heads] adds
    exp(sink_h) to the denominator, ``window`` > 0 hides keys with i - j >= window; the result is times ``out_scale``.
    ``out`` may be a column slice of a wider buffer."""
    _cuda(q, out, cache.pool, cache.block_table, ctx.positions, ctx.req_of_token, ctx.err, table, sink)
    T = q.shape[0]
    _need(q.is_contiguous() and tuple(q.shape) == (T, nh * D), "q must be contiguous [T, heads*D]")
    _need(tuple(out.shape) == (T, nh * Dv) and out.stride(1) == 1 and out.dtype == q.dtype, "out must be row-major [T, heads*Dv] of q's type")
    pool, bt = cache.pool, cache.block_table
    _need(pool.dtype == q.dtype and pool.is_contiguous() and pool[0].numel() == nkv * cache.page_size * (D + Dv),
          "the cache pages do not fit the head sizes or the type of q")
    table_len = 0
    if table is not None:
        _need(table.dtype == torch.float32 and table.dim() == 2 and table.shape[0] == nh and table.is_contiguous(),
              "the distance table must be float32 [heads, n]")
        table_len = table.shape[1]
    if sink is not None:
        _need(sink.dtype == torch.float32 and sink.numel() == nh and sink.is_contiguous(), "the sinks must be float32 [heads]")
    f = _fn("softmax_attention", "airun_softmax_attention",
            [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_float, c_void_p, c_void_p])
    _check(f(_p(q), _p(out), _row_stride(out), _p(pool), _dt(q), _p(bt), bt.stride(0), _p(ctx.positions), _p(ctx.req_of_token), T,
             int(ctx.num_reqs), pool.shape[0], int(cache.page_size), nh, nkv, D, Dv, float(scale), _p(table), int(table_len),
             _p(sink), int(window), float(out_scale), _p(ctx.err), _stream()), "softmax_attention")


# ---------------------------------------------------------------- products
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on the CUDA cores, float32 accumulation."""
    _cuda(a, w, out)
    _need(a.dim() == 2 and w.dim() == 2 and out.dim() == 2, "gemm takes 2-d tensors")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(out.shape) == (M, N), f"gemm shapes do not agree: {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _need(a.dtype == w.dtype, "gemm operands must share a type")
    f = _fn("gemm_simt", "airun_gemm_simt",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
             c_longlong, c_longlong, c_longlong, c_void_p])
    _check(f(_p(a), _dt(a), _p(w), _dt(w), _p(out), _dt(out), M, N, K,
             a.stride(0) if M > 1 else max(K, a.stride(0)), w.stride(0) if N > 1 else max(K, w.stride(0)),
             out.stride(0) if M > 1 else max(N, out.stride(0)), _stream()), "gemm_simt")


def gemm_simt_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[:, b, :] = a[:, b, :] @ w[b]^T for every b: a [M, B, K], w [B, N, K], out [M, B, N]; a and out may be
    views whose rows and batches are strided (column slices of wider buffers), their last axis is contiguous."""
    _cuda(a, w, out)
    _need(a.dim() == 3 and w.dim() == 3 and out.dim() == 3, "the batched product takes 3-d tensors")
    M, B, K = a.shape
    N = w.shape[1]
    _need(w.shape[0] == B and w.shape[2] == K and tuple(out.shape) == (M, B, N), "batched product shapes do not agree")
    _need(a.stride(2) == 1 and w.stride(2) == 1 and out.stride(2) == 1, "operands must be row-major in their last axis")
    _need(a.dtype == w.dtype, "operands must share a type")
    f = _fn("gemm_simt", "airun_gemm_simt_batched",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
             c_int, c_longlong, c_longlong, c_longlong, c_void_p])
    lda = a.stride(0) if M > 1 else max(K, a.stride(0))
    ldc = out.stride(0) if M > 1 else max(N, out.stride(0))
    _check(f(_p(a), _dt(a), _p(w), _dt(w), _p(out), _dt(out), M, N, K, lda, w.stride(1) if N > 1 else max(K, w.stride(1)), ldc,
             B, a.stride(1), w.stride(0), out.stride(1), _stream()), "gemm_simt_batched")


def gemm_simt_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, seg: torch.Tensor) -> None:
    """Rows seg[e] .. seg[e+1]-1 of a [M, K] times w[e]^T (w [E, N, K]) into the same rows of out [M, N]; ``seg`` is
    int32 [E + 1] on the device.  Rows from seg[E] on are left as they are."""
    _cuda(a, w, out, seg)
    _need(a.dim() == 2 and w.dim() == 3 and out.dim() == 2 and a.is_contiguous() and w.is_contiguous() and out.is_contiguous(),
          "the grouped product takes contiguous a [M, K], w [E, N, K], out [M, N]")
    M, K = a.shape
    E, N = w.shape[0], w.shape[1]
    _need(w.shape[2] == K and tuple(out.shape) == (M, N) and a.dtype == w.dtype, "grouped product shapes or types do not agree")
    _need(seg.dtype == torch.int32 and seg.numel() >= E + 1 and seg.is_contiguous(), "seg must be int32 [E + 1]")
    f = _fn("gemm_simt", "airun_gemm_simt_grouped",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
             c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_p(a), _dt(a), _p(w), _dt(w), _p(out), _dt(out), M, N, K, K, K, N, _p(seg), E, N * K, _stream()),
           "gemm_simt_grouped")


# ---------------------------------------------------------------- recurrent mixers with a matrix state
def short_conv(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, tail_off: int, ctx, out: torch.Tensor,
               n_unit_heads: int, q_heads: int, unit_dim: int, unit_eps: float, q_scale: float) -> None:
    """out[t, c] = silu(sum_j weight[c, j] * x[t - (taps-1) + j, c]) over the rows of each request in order; rows
    before a request's first row of this step come from state[slot, tail_off:] viewed as [taps-1, C].  The first
    ``n_unit_heads`` heads of ``unit_dim`` channels are made unit vectors, the first ``q_heads`` of them times
    ``q_scale``.  ``x`` float32 [T, C] (a column slice is fine), ``state`` float32 [slots, n]."""
    _cuda(x, weight, state, out)
    _rows_f32(x, "x")
    T, C = x.shape
    _need(weight.dtype == torch.float32 and weight.dim() == 2 and weight.shape[0] == C and weight.is_contiguous(),
          "the convolution's weight must be float32 [C, taps]")
    taps = weight.shape[1]
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and tail_off + (taps - 1) * C <= state.shape[1],
          "state must be float32 [slots, n] with room for the tail")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (T, C) and out.is_contiguous(), "out must be float32 [T, C]")
    f = _fn("recurrent_state", "airun_short_conv",
            [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p])
    _check(f(_p(x), _row_stride(x), _p(weight), taps, _p(state), state.stride(0), int(tail_off), state.shape[0],
             _p(ctx.req_of_token), _p(ctx.cu_tokens), _p(ctx.state_slots), int(ctx.num_reqs), _p(out), T, C, int(n_unit_heads),
             int(q_heads), int(unit_dim), float(unit_eps), float(q_scale), _p(ctx.err), _stream()), "short_conv")


def token_shift(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, prev_off: int, ctx, out: torch.Tensor) -> None:
    """out[s, t] = x[t] + (x[t-1] - x[t]) * mu[s] in out's type; the row before a request's first row of this step
    is state[slot, prev_off : prev_off + W].  x float32 [T, W], mu float32 [S, W], out [S, T, W]."""
    _cuda(x, mu, state, out)
    _need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "x must be contiguous float32 [T, W]")
    T, W = x.shape
    _need(mu.dtype == torch.float32 and mu.dim() == 2 and mu.shape[1] == W and mu.is_contiguous(), "mu must be float32 [S, W]")
    S = mu.shape[0]
    _need(tuple(out.shape) == (S, T, W) and out.is_contiguous(), "out must be contiguous [S, T, W]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and prev_off + W <= state.shape[1],
          "state must be float32 [slots, n] with room for the row")
    f = _fn("recurrent_state", "airun_token_shift",
            [c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
             c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(x), _p(mu), S, _p(state), state.stride(0), int(prev_off), state.shape[0], _p(ctx.req_of_token), _p(ctx.cu_tokens),
             _p(ctx.state_slots), int(ctx.num_reqs), _p(out), _dt(out), T, W, _p(ctx.err), _stream()), "token_shift")


RECURRENCE_DELTA, RECURRENCE_WKV = 0, 1


def recurrent_state(mode: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, state: torch.Tensor, ctx,
                    out: torch.Tensor, heads: int, kv_rep: int, D: int, Dv: int, beta: Optional[torch.Tensor] = None,
                    bonus: Optional[torch.Tensor] = None, tail_src: Optional[torch.Tensor] = None, tail_off: int = 0,
                    tail_rows: int = 0) -> None:
    """The delta rule (RECURRENCE_DELTA: q, k [T, heads/kv_rep * D], v [T, heads*Dv], decay g [T, heads*D], beta
    [T, heads] BEFORE its sigmoid) or the time mix with a bonus (RECURRENCE_WKV: r, k, v, decay [T, heads*D], bonus [heads, D]) over the
    rows of every request in order, on state[slot, : heads*D*Dv] viewed as [heads, D, Dv]; out float32 [T, heads*Dv].
    With ``tail_rows`` the last rows of (state[slot, tail_off:] as [tail_rows, C], then this step's rows of
    ``tail_src`` [T, C]) are kept there for the next step."""
    _cuda(q, k, v, g, state, out, beta, bonus, tail_src)
    for t_, name in ((q, "q"), (k, "k"), (v, "v"), (g, "g")):
        _rows_f32(t_, name)
    T = q.shape[0]
    _need(q.shape[1] == heads // kv_rep * D and k.shape[1] == q.shape[1] and v.shape[1] == heads * Dv and g.shape[1] == heads * D,
          "q, k, v or the decay has the wrong width")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= heads * D * Dv,
          "state must be float32 [slots, >= heads*D*Dv]")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (T, heads * Dv) and out.is_contiguous(), "out must be float32 [T, heads*Dv]")
    bs = 0
    if beta is not None:
        _rows_f32(beta, "beta")
        _need(beta.shape[1] == heads, "beta must be [T, heads]")
        bs = _row_stride(beta)
    if bonus is not None:
        _need(bonus.dtype == torch.float32 and bonus.numel() == heads * D and bonus.is_contiguous(), "bonus must be float32 [heads, D]")
    tw = ts = 0
    if tail_rows:
        _rows_f32(tail_src, "tail_src")
        tw, ts = tail_src.shape[1], _row_stride(tail_src)
        _need(tail_off + tail_rows * tw <= state.shape[1], "the tail does not fit the state")
    f = _fn("recurrent_state", "airun_recurrent_state",
            [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_longlong, c_void_p, c_longlong,
             c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
             c_longlong, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p])
    long_chains = 1 if T > 2 * int(ctx.num_reqs) else 0          # requests bring many tokens each, not one
    _check(f(int(mode), _p(q), _p(k), _p(v), _p(g), _row_stride(q), _row_stride(k), _row_stride(v), _row_stride(g), _p(beta), bs,
             _p(bonus), _p(state), state.stride(0), state.shape[0], _p(ctx.cu_tokens), _p(ctx.state_slots), int(ctx.num_reqs),
             _p(out), heads, kv_rep, D, Dv, _p(tail_src), ts, int(tail_off), int(tail_rows), tw, long_chains, _p(ctx.err),
             _stream()), "recurrent_state")


# ---------------------------------------------------------------- attention over a cached latent
def _latent_pool(pool: torch.Tensor, page_size: int, row: int) -> int:
    _need(pool.is_contiguous() and pool.dim() >= 2 and pool[0].numel() == page_size * row,
          f"a latent cache page must hold {page_size} rows of {row}")
    return pool.shape[0]


def latent_prepare(proj: torch.Tensor, wq: torch.Tensor, wkv: Optional[torch.Tensor], eps: float, cq: torch.Tensor,
                   R: int, rd: int, rot_dims: int, inv_freq: Optional[torch.Tensor], rot_mult: float, cache, ctx,
                   store: bool) -> None:
    """cq = rmsnorm(proj[:, :q_rank]) * wq; with ``store`` the token's cache row becomes
    [rmsnorm(proj[:, q_rank : q_rank+R]) * wkv | rotate(proj[:, q_rank+R : q_rank+R+rd])]."""
    _cuda(proj, wq, wkv, cq, inv_freq)
    _rows_f32(proj, "proj")
    T, q_rank = cq.shape
    _need(cq.is_contiguous() and proj.shape[0] == T and proj.shape[1] >= q_rank + ((R + rd) if store else 0), "proj is too narrow")
    num_pages = max_blocks = 0
    pool = bt = None
    if store:
        pool, bt = cache.pool, cache.block_table
        num_pages = _latent_pool(pool, cache.page_size, R + rd)
        _need(pool.dtype == cq.dtype, "the latent query and the cache pages must share a type")
        max_blocks = bt.stride(0)
    f = _fn("latent_attention", "airun_latent_prepare",
            [c_void_p, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float,
             c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(proj), _row_stride(proj), _p(wq), _p(wkv), float(eps), _p(cq), _dt(cq), q_rank, R, rd, rot_dims, _p(inv_freq),
             float(rot_mult), _p(pool), _p(bt), max_blocks, _p(ctx.positions), _p(ctx.req_of_token), T, int(ctx.num_reqs),
             num_pages, int(cache.page_size), 1 if store else 0, _p(ctx.err), _stream()), "latent_prepare")


def latent_query(q: torch.Tensor, qn: torch.Tensor, qlat: torch.Tensor, H: int, D: int, R: int, rd: int, rot_dims: int,
                 inv_freq: Optional[torch.Tensor], rot_mult: float, ctx) -> None:
    """q float32 [T, H*(D+rd)] -> qn [T, H*D] (the unrotated parts) and the rotated parts, turned by each token's
    position, into qlat[t, h, R:] (qlat [T, H*(R+rd)])."""
    _cuda(q, qn, qlat, inv_freq)
    T = q.shape[0]
    _need(q.dtype == torch.float32 and tuple(q.shape) == (T, H * (D + rd)) and q.is_contiguous(), "q must be float32 [T, H*(D+rd)]")
    _need(tuple(qn.shape) == (T, H * D) and qn.is_contiguous() and tuple(qlat.shape) == (T, H * (R + rd)) and qlat.is_contiguous()
          and qn.dtype == qlat.dtype, "qn / qlat must be contiguous [T, H*D] / [T, H*(R+rd)] of one type")
    f = _fn("latent_attention", "airun_latent_query",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p,
             c_void_p])
    _check(f(_p(q), _p(qn), _p(qlat), _dt(qn), T, H, D, R, rd, rot_dims, _p(inv_freq), float(rot_mult), _p(ctx.positions),
             _p(ctx.req_of_token), _stream()), "latent_query")


def latent_attention(qlat: torch.Tensor, out: torch.Tensor, cache, ctx, H: int, R: int, rd: int, scale: float, window: int,
                     sink: Optional[torch.Tensor]) -> None:
    """out[t, h] = sum_j p_j c_j over the cached rows [c | kr] each token sees (0 <= pos - j < window, or all with
    window 0), p the softmax of scale * qlat[t, h] . [c_j | kr_j] with exp(sink[h]) added to its denominator."""
    _cuda(qlat, out, sink)
    T = qlat.shape[0]
    _need(tuple(qlat.shape) == (T, H * (R + rd)) and qlat.is_contiguous() and tuple(out.shape) == (T, H * R) and out.is_contiguous()
          and out.dtype == qlat.dtype, "qlat / out must be contiguous [T, H*(R+rd)] / [T, H*R] of one type")
    num_pages = _latent_pool(cache.pool, cache.page_size, R + rd)
    _need(cache.pool.dtype == qlat.dtype, "the query and the cache pages must share a type")
    _need(R + rd <= 640, "cached rows above 640 elements are beyond the kernel")
    if sink is not None:
        _need(sink.dtype == torch.float32 and sink.numel() == H and sink.is_contiguous(), "sink must be float32 [H]")
    f = _fn("latent_attention", "airun_latent_attention",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_float, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_p(qlat), _p(out), _dt(qlat), _p(cache.pool), _p(cache.block_table), cache.block_table.stride(0), _p(ctx.positions),
             _p(ctx.req_of_token), T, int(ctx.num_reqs), num_pages, int(cache.page_size), H, R, rd, float(scale), int(window),
             _p(sink), _p(ctx.err), _stream()), "latent_attention")


# ---------------------------------------------------------------- routed experts
def moe_route(logits: torch.Tensor, top: int, softmax_scores: bool, renorm: bool, req_of_token: torch.Tensor,
              ids: torch.Tensor, wts: torch.Tensor, rank: torch.Tensor, counts: torch.Tensor, seg: torch.Tensor,
              bias: Optional[torch.Tensor] = None) -> None:
    """ids / wts [T, top]: every token's ``top`` experts by score (sigmoid or softmax of the router's ``logits``
    [T, E], float32) and their weights; rank [T, top]: the row's place among its expert's rows; seg [E + 1]: where each
    expert's rows begin.  ``counts`` (int32 [E]) must be zero on entry.  ``bias`` (float32 [E]) is added to the logits first."""
    _cuda(logits, req_of_token, ids, wts, rank, counts, seg, bias)
    _rows_f32(logits, "logits")
    T, E = logits.shape
    _need(E <= 1024 and 1 <= top <= E, "1 to 1024 experts, top of them a token")
    for t_, dt in ((ids, torch.int32), (wts, torch.float32), (rank, torch.int32)):
        _need(t_.dtype == dt and t_.numel() >= T * top and t_.is_contiguous(), "ids / wts / rank must be [T, top]")
    _need(counts.dtype == torch.int32 and counts.numel() >= E and seg.dtype == torch.int32 and seg.numel() >= E + 1,
          "counts / seg must be int32 [E] / [E + 1]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == E and bias.is_contiguous(), "the router's bias must be float32 [E]")
    f = _fn("moe", "airun_moe_route",
            [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(logits), _row_stride(logits), _p(bias), T, E, int(top), 1 if softmax_scores else 0, 1 if renorm else 0, _p(req_of_token),
             _p(ids), _p(wts), _p(rank), _p(counts), _p(seg), _stream()), "moe_route")


def moe_scatter(h: torch.Tensor, top: int, ids, wts, rank, seg, scale_input: bool, xs: torch.Tensor, row_of: torch.Tensor,
                num_real: int = 1 << 30) -> None:
    """xs[seg[e] + rank] = h[t] (times the weight with ``scale_input``) for each of the token's experts; row_of [T, top]
    keeps the row (-1 for an expert id of ``num_real`` or more: an expert without matrices, which gets no row)."""
    _cuda(h, xs, row_of)
    T, W = h.shape
    _need(h.is_contiguous() and xs.is_contiguous() and tuple(xs.shape) == (T * top, W) and xs.dtype == h.dtype,
          "xs must be contiguous [T*top, W] of h's type")
    _need(row_of.dtype == torch.int32 and row_of.numel() >= T * top, "row_of must be int32 [T, top]")
    f = _fn("moe", "airun_moe_scatter",
            [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_p(h), _dt(h), T, W, int(top), _p(ids), _p(wts), _p(rank), _p(seg), 1 if scale_input else 0, _p(xs), _p(row_of),
             int(num_real), _stream()), "moe_scatter")


def moe_combine(ys: torch.Tensor, top: int, ids, wts, row_of, scale_output: bool, out: torch.Tensor,
                passthrough: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum over the token's experts, in the order chosen, of ys[row] (times the weight with ``scale_output``);
    an expert without a row (row_of -1) contributes ``passthrough[t]``, the feed-forward's own input [T, W]."""
    _cuda(ys, out, passthrough)
    if passthrough is not None:
        _need(tuple(passthrough.shape) == tuple(out.shape) and passthrough.is_contiguous(), "passthrough must be contiguous [T, W]")
    T, W = out.shape
    _need(ys.dtype == torch.float32 and ys.is_contiguous() and tuple(ys.shape) == (T * top, W) and out.dtype == torch.float32
          and out.is_contiguous(), "ys / out must be contiguous float32 [T*top, W] / [T, W]")
    f = _fn("moe", "airun_moe_combine", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                         c_void_p])
    _check(f(_p(ys), T, W, int(top), _p(ids), _p(wts), _p(row_of), 1 if scale_output else 0, _p(out), _p(passthrough),
             _dt(passthrough) if passthrough is not None else DT_F32, _stream()), "moe_combine")


def moe_route_grouped(logits: torch.Tensor, num_real: int, top: int, groups: int, keep: int, weight_scale: float,
                      correction: Optional[torch.Tensor], req_of_token: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor,
                      rank: torch.Tensor, counts: torch.Tensor, seg: torch.Tensor) -> None:
    """Routing by softmax scores with a correction and groups (csrc/moe.cu: moe_route_grouped_kernel).  ``logits``
    float32 [T, n_out]: the first ``num_real`` outputs are experts with matrices, the rest return their input.  Scores
    are the softmax over all outputs; the choice is by score + ``correction`` inside the ``keep`` best of ``groups``
    equal runs of neighbouring outputs; weights are the chosen scores over their sum (+ 1e-20) times ``weight_scale``.
    ``counts`` (int32 [num_real]) must be zero on entry; seg [num_real + 1]."""
    _cuda(logits, correction, req_of_token, ids, wts, rank, counts, seg)
    _rows_f32(logits, "logits")
    T, n_out = logits.shape
    _need(n_out <= 1024 and 1 <= num_real <= n_out, "1 to 1024 router outputs, at least one expert with matrices")
    _need(groups >= 1 and n_out % groups == 0 and 1 <= keep <= groups and 1 <= top <= (n_out // groups) * keep,
          "the groups must divide the router's outputs and hold at least ``top`` of them")
    for t_, dt in ((ids, torch.int32), (wts, torch.float32), (rank, torch.int32)):
        _need(t_.dtype == dt and t_.numel() >= T * top and t_.is_contiguous(), "ids / wts / rank must be [T, top]")
    _need(counts.dtype == torch.int32 and counts.numel() >= num_real and seg.dtype == torch.int32 and seg.numel() >= num_real + 1,
          "counts / seg must be int32 [experts] / [experts + 1]")
    if correction is not None:
        _need(correction.dtype == torch.float32 and correction.numel() == n_out and correction.is_contiguous(),
              "the correction must be float32 [router outputs]")
    f = _fn("moe", "airun_moe_route_grouped",
            [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_void_p])
    _check(f(_p(logits), _row_stride(logits), _p(correction), T, n_out, int(num_real), int(top), int(groups), int(keep),
             float(weight_scale), _p(req_of_token), _p(ids), _p(wts), _p(rank), _p(counts), _p(seg), _stream()), "moe_route_grouped")


# ---------------------------------------------------------------- attention
def qkv_post(qkv: torch.Tensor, q_out: torch.Tensor, q_norm_w: Optional[torch.Tensor],
             k_norm_w: Optional[torch.Tensor], eps: float, positions: torch.Tensor,
             req_of_token: torch.Tensor, rope_kind: int, rotary_dim: int, inv_freq: Optional[torch.Tensor],
             pool: Optional[torch.Tensor], block_table: Optional[torch.Tensor], num_reqs: int,
             page_size: int, nh: int, nkv: int, hd: int, err: torch.Tensor,
             store: bool = True, kv_in_row: bool = True, rope_positions: Optional[torch.Tensor] = None) -> None:
    """Per-head norm, rotary encoding, q out, k/v into their pages (see csrc/qkv_post.cu).

    ``pool`` is one layer's pages [num_pages, 2, nkv, page_size, hd].  ``rope_kind``: ROPE_NONE, ROPE_NEOX
    (pair i couples dims i and i + r/2) or ROPE_INTERLEAVED (dims 2i and 2i + 1).  ``rope_positions``
    (int32 [T]): the position each row is rotated by, when that is not its place in the cache."""
    _cuda(qkv, q_out, q_norm_w, k_norm_w, positions, req_of_token, inv_freq, pool, block_table, err, rope_positions)
    if rope_positions is not None:
        _need(rope_positions.dtype == torch.int32 and rope_positions.is_contiguous() and rope_positions.shape[0] >= qkv.shape[0],
              "rope_positions must be int32 [T]")
    T = qkv.shape[0]
    width = (nh + 2 * nkv) * hd if kv_in_row else nh * hd
    _need(qkv.dtype == torch.float32 and qkv.dim() == 2 and qkv.shape[1] == width and qkv.stride(1) == 1,
          f"qkv must be float32 [T, {width}]")
    _need(tuple(q_out.shape) == (T, nh * hd) and q_out.is_contiguous(), "q_out must be [T, nh*hd]")
    _need(hd <= 256, f"head_dim {hd} is above the kernel's limit of 256")
    for w in (q_norm_w, k_norm_w):
        if w is not None:
            _need(w.dtype == torch.float32 and tuple(w.shape) == (hd,), "q/k norm weights must be float32 [head_dim]")
    _need(positions.dtype == torch.int32 and req_of_token.dtype == torch.int32
          and positions.shape[0] >= T and req_of_token.shape[0] >= T, "positions / req_of_token must be int32 [T]")
    if rope_kind != ROPE_NONE:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.shape[0] == rotary_dim // 2,
              "inv_freq must be float32 [rotary_dim/2]")
    num_pages, max_blocks = 0, 0
    do_store = bool(store and kv_in_row)
    if do_store:
        _need(pool is not None and pool.is_contiguous() and pool.dim() == 5
              and tuple(pool.shape[1:]) == (2, nkv, page_size, hd), "pool must be [pages, 2, nkv, page_size, hd]")
        _need(pool.dtype == q_out.dtype, "q and the cache pages must share a type")
        _need(block_table is not None and block_table.dtype == torch.int32 and block_table.dim() == 2
              and block_table.stride(1) == 1, "block_table must be int32 [R, max_blocks]")
        num_pages, max_blocks = pool.shape[0], block_table.stride(0)
    f = _fn("qkv_post", "airun_qkv_post",
            [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
             c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(qkv), qkv.stride(0), _p(q_out), _dt(q_out), _p(q_norm_w), _p(k_norm_w), float(eps),
             _p(positions), _p(req_of_token), T, int(rope_kind), int(rotary_dim), _p(inv_freq), _p(rope_positions),
             _p(pool), _dt(q_out), _p(block_table), max_blocks, int(num_reqs), num_pages, int(page_size),
             1 if do_store else 0, 1 if kv_in_row else 0, nh, nkv, hd, _p(err), _stream()), "qkv_post")


def attention_generic(q: torch.Tensor, out: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor,
                      positions: torch.Tensor, req_of_token: torch.Tensor, num_reqs: int,
                      nh: int, nkv: int, hd: int, scale: float, window: int, err: torch.Tensor) -> None:
    """Causal attention of every token over its request's pages, float32 arithmetic."""
    _cuda(q, out, pool, block_table, positions, req_of_token, err)
    T = q.shape[0]
    _need(tuple(q.shape) == (T, nh * hd) and q.is_contiguous() and out.shape == q.shape and out.is_contiguous()
          and out.dtype == q.dtype, "q and out must be contiguous [T, nh*hd] of one type")
    _need(hd <= 256, f"head_dim {hd} is above the kernel's limit of 256")
    _need(nh % nkv == 0, "query heads must be a multiple of KV heads")
    _need(pool.is_contiguous() and pool.dim() == 5 and pool.shape[1] == 2 and pool.shape[2] == nkv
          and pool.shape[4] == hd and pool.dtype == q.dtype, "pool must be [pages, 2, nkv, page_size, hd] of q's type")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1,
          "block_table must be int32 [R, max_blocks]")
    f = _fn("attention_generic", "airun_attention_generic",
            [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_p(q), _p(out), _dt(q), _p(pool), _dt(pool), _p(block_table), block_table.stride(0),
             _p(positions), _p(req_of_token), T, int(num_reqs), pool.shape[0], pool.shape[3],
             nh, nkv, hd, float(scale), int(window), _p(err), _stream()), "attention_generic")


# ---------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           uniform: Optional[torch.Tensor] = None) -> None:
    """out[r] = first argmax of logits[r], or a draw at temperature[r] > 0 using uniform[r]."""
    _cuda(logits, out, temperature, uniform)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "logits must be float32 [R, V]")
    R, V = logits.shape
    _need(out.dtype == torch.int32 and out.shape[0] >= R and out.is_contiguous(), "sample output must be int32 [R]")
    for t in (temperature, uniform):
        if t is not None:
            _need(t.dtype == torch.float32 and t.shape[0] >= R and t.is_contiguous(), "temperature / uniform must be float32 [R]")
    scratch = None
    if V >= 8192:
        scratch = _SAMPLE_SCRATCH.get(logits.device)
        if scratch is None or scratch.numel() < R * 128:
            scratch = torch.empty(max(R, 256) * 128, dtype=torch.int32, device=logits.device)
            _SAMPLE_SCRATCH[logits.device] = scratch
    f = _fn("sampling", "airun_sample",
            [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(logits), logits.stride(0) if R > 1 else max(V, logits.stride(0)), R, V,
             _p(temperature), _p(uniform), _p(out), _p(scratch), _stream()), "sample")


_SAMPLE_SCRATCH = {}

LARGEST_LOGITS_MAX = 512


def largest_logits(logits: torch.Tensor, rows: torch.Tensor, n: int, n_cand: int, out_ids: torch.Tensor,
                   out_vals: torch.Tensor, out_flags: torch.Tensor) -> None:
    """For the ``n`` rows ``rows[i]`` of ``logits``: out_ids[i], out_vals[i] = the ``n_cand`` largest logits with
    their ids, the largest first, equal values by ascending id (-1 / -inf beyond the row's size); out_flags[i] != 0
    when the kernel cannot vouch for the list (the caller then takes the whole row)."""
    _cuda(logits, rows, out_ids, out_vals, out_flags)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "logits must be float32 [R, V]")
    _need(1 <= n_cand <= LARGEST_LOGITS_MAX, f"1 to {LARGEST_LOGITS_MAX} candidates a row")
    _need(rows.dtype == torch.int32 and rows.numel() >= n and rows.is_contiguous(), "rows must be int32 [n]")
    _need(out_ids.dtype == torch.int32 and out_ids.is_contiguous() and out_ids.numel() >= n * n_cand
          and out_vals.dtype == torch.float32 and out_vals.is_contiguous() and out_vals.numel() >= n * n_cand
          and out_flags.dtype == torch.int32 and out_flags.numel() >= n, "candidate outputs are [n, n_cand] and [n]")
    R, V = logits.shape
    f = _fn("sampling", "airun_largest_logits",
            [c_void_p, c_longlong, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(logits), logits.stride(0) if R > 1 else max(V, logits.stride(0)), V, _p(rows), int(n), int(n_cand),
             _p(out_ids), _p(out_vals), _p(out_flags), _stream()), "largest_logits")


def describe_device_error(bits: int) -> str:
    return "; ".join(msg for b, msg in DEV_ERR_BITS.items() if bits & b) or f"unknown error bits {bits}"
